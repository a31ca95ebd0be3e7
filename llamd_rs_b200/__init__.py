"""llamd_rs_b200: B200 (sm_100a) CUDA backend for llamd's quantized MoE hot path.

`backend` mirrors the reference's device-backend crate surface over the C ABI
declared in include/llamd_cuda.h; `model` drives the resident decode model;
`synth` makes the seeded synthetic inputs the benchmarks and tests share.
"""
from . import _lib  # noqa: F401

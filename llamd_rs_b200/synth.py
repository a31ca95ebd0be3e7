"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations. They stand in for the real Qwen3MoE checkpoint,
which is not available: every tensor is random-init.

One recipe serves the CUDA path and the CPU oracle: numpy's PCG64 streams
keyed by (seed, tensor key), so any tensor -- or any single expert of a layer
-- can be regenerated independently and byte-identically.

Q6_K block (210 B): ql[128] u8 uniform, qh[64] u8 uniform, scales[16] i8
uniform in [-32, 31], d = f16(|N(0,1)| * d_scale).
Q8_0 block (34 B): d = f16(|N(0,1)| * d_scale), 32 i8 uniform in [-127, 127].
"""
from __future__ import annotations

import zlib

import numpy as np

QK_K = 256
Q6K_BLOCK_BYTES = 210
Q8_0_BLOCK_BYTES = 34


def _rng(seed: int, *key) -> np.random.Generator:
    words = [int(seed) & 0xFFFFFFFF]
    for k in key:
        words.append(zlib.crc32(str(k).encode()) & 0xFFFFFFFF)
    return np.random.Generator(np.random.PCG64(np.random.SeedSequence(words)))


def q6k_blocks(n_blocks: int, seed: int, *key, d_scale: float = 1e-3) -> np.ndarray:
    """n_blocks Q6_K blocks in the reference's byte layout, as a flat uint8 array."""
    rng = _rng(seed, "q6k", *key)
    b = rng.integers(0, 256, size=(n_blocks, Q6K_BLOCK_BYTES), dtype=np.uint8)
    sc = (b[:, 192:208] & 63).astype(np.int16) - 32
    b[:, 192:208] = sc.astype(np.int8).view(np.uint8)
    d = (np.abs(rng.standard_normal(n_blocks)).astype(np.float32) * np.float32(d_scale)).astype(np.float16)
    b[:, 208:210] = d.view(np.uint8).reshape(n_blocks, 2)
    return b.reshape(-1)


def q8_0_blocks(n_blocks: int, seed: int, *key, d_scale: float = 1e-2) -> np.ndarray:
    rng = _rng(seed, "q8_0", *key)
    b = np.zeros((n_blocks, Q8_0_BLOCK_BYTES), dtype=np.uint8)
    q = rng.integers(-127, 128, size=(n_blocks, 32), dtype=np.int8)
    b[:, 2:] = q.view(np.uint8)
    d = (np.abs(rng.standard_normal(n_blocks)).astype(np.float32) * np.float32(d_scale)).astype(np.float16)
    b[:, 0:2] = d.view(np.uint8).reshape(n_blocks, 2)
    return b.reshape(-1)


def normal_f32(n, seed: int, *key, std: float = 1.0) -> np.ndarray:
    rng = _rng(seed, "f32", *key)
    return (rng.standard_normal(n).astype(np.float32) * np.float32(std)).astype(np.float32)


def token_ids(n: int, n_vocab: int, seed: int, *key) -> np.ndarray:
    return _rng(seed, "tok", *key).integers(0, n_vocab, size=n, dtype=np.int64).astype(np.uint32)


def checksum(*arrays) -> str:
    c = 0
    for a in arrays:
        c = zlib.crc32(np.ascontiguousarray(a).view(np.uint8).reshape(-1), c)
    return f"{c & 0xFFFFFFFF:08x}"


# The architecture of the decode benchmark: Qwen3MoE, 48 layers, 128 experts.
QWEN3MOE_30B = dict(n_layer=48, n_embd=2048, n_head=32, n_head_kv=4, head_dim=128, n_expert=128, n_expert_used=8,
                    n_ff_expert=768, n_vocab=151936, rope_freq_base=1e7, rms_eps=1e-6)

# A small model of the same architecture for parity tests the oracle finishes in seconds.
TINY = dict(n_layer=2, n_embd=256, n_head=4, n_head_kv=2, head_dim=64, n_expert=8, n_expert_used=2,
            n_ff_expert=256, n_vocab=512, rope_freq_base=1e7, rms_eps=1e-6)


def expert_blocks(hp: dict, seed: int, layer: int, which: int, expert: int) -> np.ndarray:
    """One expert's Q6_K bytes. which: 0 gate, 1 up ([n_ff x n_embd]), 2 down ([n_embd x n_ff])."""
    n_blocks = hp["n_ff_expert"] * hp["n_embd"] // QK_K
    return q6k_blocks(n_blocks, seed, "layer", layer, ("gate", "up", "down")[which], expert)


def layer_weights(hp: dict, seed: int, il: int, with_experts: bool = True) -> dict:
    E, H = hp["n_embd"], hp["head_dim"]
    qd, kvd = hp["n_head"] * H, hp["n_head_kv"] * H
    lay = dict(
        attn_norm=np.ones(E, np.float32),
        attn_q=q6k_blocks(qd * E // QK_K, seed, "layer", il, "attn_q"),
        attn_k=q6k_blocks(kvd * E // QK_K, seed, "layer", il, "attn_k"),
        attn_v=q6k_blocks(kvd * E // QK_K, seed, "layer", il, "attn_v"),
        attn_q_norm=np.ones(H, np.float32),
        attn_k_norm=np.ones(H, np.float32),
        attn_out=q6k_blocks(E * qd // QK_K, seed, "layer", il, "attn_out"),
        ffn_norm=np.ones(E, np.float32),
        ffn_gate_inp=normal_f32(hp["n_expert"] * E, seed, "layer", il, "router", std=0.02),
    )
    if with_experts:
        for which, name in enumerate(("ffn_gate_exps", "ffn_up_exps", "ffn_down_exps")):
            lay[name] = np.concatenate([expert_blocks(hp, seed, il, which, e) for e in range(hp["n_expert"])])
    return lay


def make_model(hp: dict, seed: int = 0, with_experts: bool = True, n_layer: int | None = None) -> dict:
    """Random-init weights in the reference's (ggml) byte layouts; norms are 1.0,
    the router is f32 N(0, 0.02), every other linear weight is Q6_K."""
    E = hp["n_embd"]
    L = hp["n_layer"] if n_layer is None else n_layer
    return dict(
        tok_embd=q6k_blocks(hp["n_vocab"] * E // QK_K, seed, "tok_embd"),
        output_norm=np.ones(E, np.float32),
        output=q6k_blocks(hp["n_vocab"] * E // QK_K, seed, "output"),
        layers=[layer_weights(hp, seed, il, with_experts) for il in range(L)],
    )

"""CudaModel: Python handle on the resident decode model in libllamd_cuda.so.

Mirrors ``DeviceModel`` (crates/llamd-runtime/src/device.rs): ``load`` /
``load_batched``, ``forward(token, pos) -> token``, ``forward_batch``,
``logits``, ``weight_bytes``, ``hparams`` and the public knobs ``use_graph``.
Weights come as a dict of numpy arrays in the reference's byte layouts (see
``synth.make_model``), or are streamed expert by expert for models too large
to hold on the host.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import backend
from ._lib import lib

(T_TOK_EMBD, T_OUTPUT_NORM, T_OUTPUT, T_ATTN_NORM, T_ATTN_Q, T_ATTN_K, T_ATTN_V, T_ATTN_Q_NORM, T_ATTN_K_NORM,
 T_ATTN_OUT, T_FFN_NORM, T_FFN_GATE_INP, T_FFN_GATE_EXPS, T_FFN_UP_EXPS, T_FFN_DOWN_EXPS) = range(15)

_LAYER_TENSORS = dict(attn_norm=T_ATTN_NORM, attn_q=T_ATTN_Q, attn_k=T_ATTN_K, attn_v=T_ATTN_V,
                      attn_q_norm=T_ATTN_Q_NORM, attn_k_norm=T_ATTN_K_NORM, attn_out=T_ATTN_OUT, ffn_norm=T_FFN_NORM,
                      ffn_gate_inp=T_FFN_GATE_INP, ffn_gate_exps=T_FFN_GATE_EXPS, ffn_up_exps=T_FFN_UP_EXPS,
                      ffn_down_exps=T_FFN_DOWN_EXPS)
_F32 = {T_OUTPUT_NORM, T_ATTN_NORM, T_ATTN_Q_NORM, T_ATTN_K_NORM, T_FFN_NORM, T_FFN_GATE_INP}


class _Hparams(C.Structure):
    _fields_ = [(k, C.c_int32) for k in ("n_layer", "n_embd", "n_head", "n_head_kv", "head_dim", "n_expert",
                                         "n_expert_used", "n_ff_expert", "n_vocab")] + \
               [("rope_freq_base", C.c_float), ("rms_eps", C.c_float)]


def _bind():
    L = lib()
    if getattr(L, "_model_bound", False):
        return L
    vp, i32 = C.c_void_p, C.c_int
    L.llamd_model_create.restype = vp
    L.llamd_model_create.argtypes = [C.POINTER(_Hparams), i32, i32]
    L.llamd_model_free.restype = None
    L.llamd_model_free.argtypes = [vp]
    L.llamd_model_error.restype = C.c_char_p
    L.llamd_model_error.argtypes = [vp]
    L.llamd_model_set_tensor.restype = i32
    L.llamd_model_set_tensor.argtypes = [vp, i32, i32, C.c_size_t, vp, C.c_size_t]
    L.llamd_model_weight_bytes.restype = C.c_size_t
    L.llamd_model_weight_bytes.argtypes = [vp]
    L.llamd_model_set_option.restype = i32
    L.llamd_model_set_option.argtypes = [vp, C.c_char_p, i32]
    L.llamd_model_forward.restype = i32
    L.llamd_model_forward.argtypes = [vp, C.c_int32, C.c_int32, C.POINTER(C.c_int32)]
    L.llamd_model_forward_batch.restype = i32
    L.llamd_model_forward_batch.argtypes = [vp, vp, vp, i32, vp]
    L.llamd_model_logits.restype = i32
    L.llamd_model_logits.argtypes = [vp, vp, i32]
    L.llamd_model_read_trace.restype = i32
    L.llamd_model_read_trace.argtypes = [vp, vp, vp]
    L.llamd_model_read_kv.restype = i32
    L.llamd_model_read_kv.argtypes = [vp, i32, i32, i32, vp, vp]
    L.llamd_model_prefill.restype = i32
    L.llamd_model_prefill.argtypes = [vp, vp, i32, i32, C.POINTER(C.c_int32)]
    L.llamd_model_decode.restype = i32
    L.llamd_model_decode.argtypes = [vp, C.c_int32, C.c_int32, i32, vp, C.POINTER(C.c_float)]
    L.llamd_model_bench_matvecs.restype = i32
    L.llamd_model_bench_matvecs.argtypes = [vp, i32, i32, C.POINTER(C.c_float), C.POINTER(i32)]
    L.llamd_model_launches_per_pass.restype = C.c_ulonglong
    L.llamd_model_launches_per_pass.argtypes = [vp]
    L.llamd_model_profile_pass.restype = i32
    L.llamd_model_profile_pass.argtypes = [vp, C.c_int32, C.c_int32, vp]
    L.llamd_cuda_ep_unique_id.restype = i32
    L.llamd_cuda_ep_unique_id.argtypes = [vp]
    L.llamd_cuda_ep_init.restype = i32
    L.llamd_cuda_ep_init.argtypes = [i32, i32, vp]
    L.llamd_cuda_ep_finalize.restype = None
    L.llamd_cuda_ep_finalize.argtypes = []
    L.llamd_cuda_ep_rank.restype = i32
    L.llamd_cuda_ep_world.restype = i32
    L.llamd_cuda_ep_init_local.restype = i32
    L.llamd_cuda_ep_init_local.argtypes = [i32, i32]
    L.llamd_cuda_ep_set_timeout_ms.restype = None
    L.llamd_cuda_ep_set_timeout_ms.argtypes = [i32]
    L.llamd_model_ep_status.restype = i32
    L.llamd_model_ep_status.argtypes = [vp]
    L.llamd_model_ep_p2p_buffers.restype = i32
    L.llamd_model_ep_p2p_buffers.argtypes = [vp, vp]
    L.llamd_model_verify.restype = i32
    L.llamd_model_verify.argtypes = [vp, vp, i32, i32, vp]
    L.llamd_model_resident_profile.restype = i32
    L.llamd_model_resident_profile.argtypes = [vp, vp]
    L.llamd_model_ep_tile_cap.restype = i32
    L.llamd_model_ep_tile_cap.argtypes = [vp]
    L.llamd_model_ep_p2p_attach_ptrs.restype = i32
    L.llamd_model_ep_p2p_attach_ptrs.argtypes = [vp, vp, i32]
    L._model_bound = True
    return L


EP_P2P_RECORD = 640  # LLAMD_EP_P2P_RECORD: ten 64-byte IPC handles


def ep_init(rank: int, world: int, share) -> None:
    """Join the expert-parallel communicator. `share(bytes_or_None) -> bytes`
    hands rank 0's 128-byte id to every rank (e.g. a torch.distributed/gloo
    broadcast); call after backend.set_device and before creating the model."""
    L = _bind()
    buf = C.create_string_buffer(128)
    if rank == 0 and L.llamd_cuda_ep_unique_id(buf) != 0:
        raise backend.Other("ep unique id: " + backend._last_error())
    ident = share(bytes(buf.raw) if rank == 0 else None)
    if len(ident) != 128:
        raise backend.Malformed("ep id must be 128 bytes")
    if L.llamd_cuda_ep_init(rank, world, C.create_string_buffer(ident, 128)) != 0:
        raise backend.Other("ep init: " + backend._last_error())


def ep_init_local(rank: int, world: int) -> None:
    """Rank and world without a communicator: only the peer-memory form can then be used (attach before the first pass)."""
    if _bind().llamd_cuda_ep_init_local(rank, world) != 0:
        raise backend.Other("ep init (local): " + backend._last_error())


def ep_set_timeout_ms(ms: int) -> None:
    """How long the host waits for other ranks (communicator set-up, a pass with collectives) before it gives up."""
    _bind().llamd_cuda_ep_set_timeout_ms(int(ms))


def ep_finalize() -> None:
    _bind().llamd_cuda_ep_finalize()


class CudaModel:
    def __init__(self, hp: dict, max_kv: int, max_seq: int = 1):
        if max_kv == 0:
            raise backend.Malformed("device model: max_kv of 0")
        if max_seq == 0 or max_seq > backend.MAX_BATCH:
            raise backend.Malformed(f"device model: max_seq {max_seq} outside 1..={backend.MAX_BATCH}")
        if not backend.available():
            raise backend.Unsupported("cuda: no device present (there is no CPU fallback)")
        self._L = _bind()
        self.hp = dict(hp)
        h = _Hparams()
        for k, _ in _Hparams._fields_:
            setattr(h, k, hp[k])
        self.max_kv, self.max_seq = max_kv, max_seq
        self._h = self._L.llamd_model_create(C.byref(h), max_kv, max_seq)
        if not self._h:
            raise backend.Other("model create failed: " + backend._last_error())
        self._use_graph = True

    # -- loading -----------------------------------------------------------
    @classmethod
    def load(cls, hp: dict, weights: dict, max_kv: int) -> "CudaModel":
        return cls.load_batched(hp, weights, max_kv, 1)

    @classmethod
    def load_batched(cls, hp: dict, weights: dict, max_kv: int, max_seq: int) -> "CudaModel":
        m = cls(hp, max_kv, max_seq)
        m.set_tensor(-1, T_TOK_EMBD, weights["tok_embd"])
        m.set_tensor(-1, T_OUTPUT_NORM, weights["output_norm"])
        if weights.get("output") is not None:
            m.set_tensor(-1, T_OUTPUT, weights["output"])
        for il, lay in enumerate(weights["layers"]):
            for name, tid in _LAYER_TENSORS.items():
                if lay.get(name) is not None:
                    m.set_tensor(il, tid, lay[name])
        return m

    @classmethod
    def load_synthetic(cls, hp: dict, seed: int, max_kv: int, max_seq: int = 1) -> "CudaModel":
        """Random-init weights streamed tensor by tensor (expert by expert), so
        a 24 GB model never has to sit in host memory. Byte-identical to
        ``load_batched(hp, synth.make_model(hp, seed), ...)``."""
        from . import synth

        m = cls(hp, max_kv, max_seq)
        E = hp["n_embd"]
        m.set_tensor(-1, T_TOK_EMBD, synth.q6k_blocks(hp["n_vocab"] * E // backend.QK_K, seed, "tok_embd"))
        m.set_tensor(-1, T_OUTPUT_NORM, np.ones(E, np.float32))
        m.set_tensor(-1, T_OUTPUT, synth.q6k_blocks(hp["n_vocab"] * E // backend.QK_K, seed, "output"))
        for il in range(hp["n_layer"]):
            lay = synth.layer_weights(hp, seed, il, with_experts=False)
            for name, tid in _LAYER_TENSORS.items():
                if name in lay:
                    m.set_tensor(il, tid, lay[name])
            # with expert parallelism only this rank's experts are generated and sent
            world, rank = m._L.llamd_cuda_ep_world(), m._L.llamd_cuda_ep_rank()
            per = hp["n_expert"] // world
            for which in range(3):
                for e in range(rank * per, (rank + 1) * per):
                    m.set_expert(il, which, e, synth.expert_blocks(hp, seed, il, which, e))
        return m

    @classmethod
    def open_gguf(cls, path, max_kv: int, max_seq: int = 1) -> "CudaModel":
        """``DeviceModel::load_batched(&Model::open(path)?, max_kv, max_seq)`` (crates/llamd-models/src/model.rs:108-131,
        crates/llamd-runtime/src/device.rs:270): the file is mapped by the library and its tensors go to the device
        from the mapping. Raises with the reference's error kinds."""
        from . import gguf

        if max_seq == 0 or max_seq > backend.MAX_SEQ:
            raise backend.Malformed(f"device model: max_seq {max_seq} outside 1..={backend.MAX_SEQ}")
        with gguf.Gguf.open(path) as g:
            hp = g.hparams()
            g.verify_present()
            if hp["arch"] != "qwen3moe":
                raise backend.Unsupported("device model: only MoE models are wired up; a dense FFN has no expert path")
            if max_kv == 0:
                raise backend.Malformed("device model: max_kv of 0")
            if not backend.available():
                raise backend.Unsupported("cuda: no device present (there is no CPU fallback)")
            kind, err = C.c_int(0), C.create_string_buffer(512)
            h = g._L.llamd_model_load_gguf(g._h, max_kv, max_seq, C.byref(kind), err, 512)
            if not h:
                gguf.raise_kind(kind.value, err.value.decode(errors="replace"))
        m = cls.__new__(cls)
        m._L = _bind()
        m.hp = {k: hp[k] for k, _ in _Hparams._fields_}
        m.max_kv, m.max_seq = max_kv, max_seq
        m._h = h
        m._use_graph = True
        return m

    def set_tensor(self, layer: int, which: int, data, first_block: int = 0) -> None:
        if which in _F32:
            a = np.ascontiguousarray(data, dtype=np.float32).ravel()
            count = a.size
        else:
            a = np.ascontiguousarray(data, dtype=np.uint8).ravel()
            if a.size % backend.Q6K_BLOCK_BYTES:
                raise backend.Malformed(f"tensor of {a.size} bytes is not whole Q6_K blocks")
            count = a.size // backend.Q6K_BLOCK_BYTES
        rc = self._L.llamd_model_set_tensor(self._h, layer, which, first_block, a.ctypes.data_as(C.c_void_p), count)
        if rc != 0:
            raise backend.Malformed("set_tensor: " + self._err())

    def set_expert(self, layer: int, which: int, expert: int, data) -> None:
        """which: 0 gate, 1 up, 2 down. Expert e is a contiguous block range
        (crates/llamd-models/src/model.rs:182-227)."""
        per = self.hp["n_ff_expert"] * self.hp["n_embd"] // backend.QK_K
        self.set_tensor(layer, (T_FFN_GATE_EXPS, T_FFN_UP_EXPS, T_FFN_DOWN_EXPS)[which], data, expert * per)

    # -- running -----------------------------------------------------------
    def _err(self) -> str:
        return self._L.llamd_model_error(self._h).decode(errors="replace")

    @property
    def use_graph(self) -> bool:
        return self._use_graph

    @use_graph.setter
    def use_graph(self, v: bool) -> None:
        self._use_graph = bool(v)
        self._L.llamd_model_set_option(self._h, b"use_graph", int(bool(v)))

    @property
    def prefill_tile(self) -> int:
        return getattr(self, "_prefill_tile", 512)

    @prefill_tile.setter
    def prefill_tile(self, v: int) -> None:
        if self._L.llamd_model_set_option(self._h, b"prefill_tile", int(v)) != 0:
            raise backend.Malformed(f"prefill_tile {v} outside 1..4096")
        self._prefill_tile = int(v)

    def set_prefill_gemm(self, on) -> None:
        """True / 1 (default): the prefill tile's matmuls run on the integer tensor path; False / 0: dp4a, 8 tokens
        per pass (both bit-identical to decode); 2: tcgen05 on f16 pairs, tolerance level."""
        self._L.llamd_model_set_option(self._h, b"prefill_gemm", int(on))

    def set_option(self, name: str, value: int) -> None:
        """llamd_model_set_option by name: use_graph, pdl, prefetch, trace, prefill_tile, prefill_gemm, prefill_attn."""
        if self._L.llamd_model_set_option(self._h, name.encode(), int(value)) != 0:
            raise backend.Malformed(f"set_option {name}={value}: " + self._err())

    def ep_p2p_attach(self, gather) -> None:
        """Expert parallelism over peer memory (no collective in the pass): exchange the IPC handles of every rank's
        request and expert-output buffers and counters and map the peers' buffers. `gather(bytes) -> list[bytes]` returns every rank's
        record in rank order (e.g. torch.distributed.all_gather_object over gloo). Every rank must call it, and the
        ranks should meet at a barrier before the first pass: a rank waits a few seconds for its peers, not forever."""
        buf = C.create_string_buffer(EP_P2P_RECORD)
        if self._L.llamd_model_ep_p2p_export(self._h, buf) != 0:
            raise backend.Other("ep_p2p export: " + (self._err() or backend._last_error()))
        records = gather(bytes(buf.raw))
        if any(len(r) != EP_P2P_RECORD for r in records):
            raise backend.Malformed(f"ep_p2p: every rank's record must be {EP_P2P_RECORD} bytes")
        blob = b"".join(records)
        if self._L.llamd_model_ep_p2p_attach(self._h, C.create_string_buffer(blob, len(blob)), len(records)) != 0:
            raise backend.Other("ep_p2p attach: " + (self._err() or backend._last_error()))

    def ep_p2p_buffers(self):
        """This rank's shared buffers as device addresses: expert outputs, arrival counter, gathered ids / scales / quants,
        dispatch counter (decode pass); expert outputs, gathered quants / scales / ids (prefill tile)."""
        out = (C.c_void_p * (EP_P2P_RECORD // 64))()
        if self._L.llamd_model_ep_p2p_buffers(self._h, out) != 0:
            raise backend.Other("ep_p2p buffers: " + (self._err() or backend._last_error()))
        return [int(v or 0) for v in out]

    def ep_p2p_attach_ptrs(self, table) -> None:
        """table: [world][EP_P2P_RECORD // 64] device addresses in the order of ep_p2p_buffers (this rank's own row is ignored)."""
        world = len(table)
        flat = (C.c_void_p * (EP_P2P_RECORD // 64 * world))(*[int(v) for row in table for v in row])
        if self._L.llamd_model_ep_p2p_attach_ptrs(self._h, flat, world) != 0:
            raise backend.Other("ep_p2p attach: " + (self._err() or backend._last_error()))

    RESIDENT_PHASES = ("A image + qkv rows", "barrier", "B1 qk-norm rope kv-store scores", "barrier", "B2 softmax values",
                       "barrier", "C quant + attn_out rows", "barrier", "D router", "barrier", "E gate/up rows",
                       "barrier", "F down rows", "barrier", "A combine", "A norm + quant", "-", "D add + norm + quant + image",
                       "E logits load", "E route", "E prefetch of down rows", "F silu + quant + image",
                       "A norm: squares", "A norm: chain", "A norm: scale")

    def resident_profile_raw(self) -> list:
        """The 32 counters of the resident kernel's CTA 0 since set_option("resident_profile", 1): nanoseconds per phase in
        RESIDENT_PHASES' order; [30] SM cycles and [31] nanoseconds of the whole kernel, summed over the tokens."""
        out = (C.c_ulonglong * 32)()
        if self._L.llamd_model_resident_profile(self._h, out) != 0:
            raise backend.Other("resident profile: " + (self._err() or backend._last_error()))
        return [int(v) for v in out]

    def resident_profile(self) -> dict:
        """Nanoseconds per phase accumulated by the resident kernel's CTA 0 since set_option("resident_profile", 1)."""
        out = self.resident_profile_raw()
        return {f"{i:02d} {name}": out[i] for i, name in enumerate(self.RESIDENT_PHASES)}

    def ep_tile_cap(self) -> int:
        """Tokens per rank and tile of expert-parallel prefill (0 until the buffers have been shared)."""
        return int(self._L.llamd_model_ep_tile_cap(self._h))

    def ep_status(self) -> int:
        return int(self._L.llamd_model_ep_status(self._h))

    def set_prefill_attn(self, on: bool) -> None:
        """True (default): a prefill tile's attention runs on the register-tiled kernels; False: the per-token ones."""
        self._L.llamd_model_set_option(self._h, b"prefill_attn", int(on))

    def set_trace(self, on: bool) -> None:
        if self._L.llamd_model_set_option(self._h, b"trace", int(on)) != 0:
            raise backend.Other("trace buffers: " + self._err())

    def forward(self, token: int, pos: int) -> int:
        if pos >= self.max_kv:
            raise backend.Malformed(f"device forward: position {pos} beyond the {self.max_kv} allocated")
        out = C.c_int32(-1)
        if self._L.llamd_model_forward(self._h, int(token), int(pos), C.byref(out)) != 0:
            raise backend.Other("forward: " + self._err())
        return int(out.value)

    def forward_batch(self, tokens, positions) -> np.ndarray:
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        p = np.ascontiguousarray(positions, dtype=np.int32)
        if t.size != p.size or t.size == 0 or t.size > self.max_seq:
            raise backend.Malformed(f"forward_batch: {t.size} tokens, {p.size} positions, max_seq {self.max_seq}")
        out = np.zeros(t.size, dtype=np.int32)
        rc = self._L.llamd_model_forward_batch(self._h, t.ctypes.data_as(C.c_void_p), p.ctypes.data_as(C.c_void_p), t.size,
                                               out.ctypes.data_as(C.c_void_p))
        if rc != 0:
            raise backend.Other("forward_batch: " + self._err())
        return out

    def prefill(self, tokens, base_pos: int = 0) -> int:
        """VulkanModel::prefill (crates/llamd-runtime/src/vulkan_model.rs:877-907):
        run a whole prompt, return the greedy token after its last position."""
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        if t.size == 0:
            raise backend.Malformed("prefill: empty prompt")
        out = C.c_int32(-1)
        if self._L.llamd_model_prefill(self._h, t.ctypes.data_as(C.c_void_p), t.size, int(base_pos), C.byref(out)) != 0:
            raise backend.Other("prefill: " + self._err())
        return int(out.value)

    def verify(self, tokens, base_pos: int = 0) -> np.ndarray:
        """out[i] = the greedy token after tokens[0..=i] (llamd_model_verify): every drafted token checked by the model."""
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        if t.size == 0 or base_pos + t.size > self.max_kv:
            raise backend.Malformed("verify: empty, or positions beyond the allocated cache")
        out = np.zeros(t.size, dtype=np.int32)
        if self._L.llamd_model_verify(self._h, t.ctypes.data_as(C.c_void_p), t.size, int(base_pos), out.ctypes.data_as(C.c_void_p)) != 0:
            raise backend.Other("verify: " + self._err())
        return out

    def speculative_decode(self, first_token: int, start_pos: int, n: int, draft, max_draft: int = 8):
        """n greedy tokens after `first_token` at `start_pos`, with `draft(context_tokens, k) -> k guessed tokens` proposing
        and the model verifying every guess. Returns (tokens, passes): the tokens equal plain greedy decode's whatever
        the drafter says; only the number of passes changes."""
        out, cur, pos, passes = [], int(first_token), int(start_pos), 0
        while len(out) < n:
            k = min(max_draft, n - len(out) - 1, self.max_kv - pos - 1)
            guess = [int(g) for g in draft(out, k)] if k > 0 else []
            got = self.verify([cur] + guess, pos)
            passes += 1
            accepted = 0
            while accepted < len(guess) and guess[accepted] == int(got[accepted]):
                accepted += 1
            new = [int(t) for t in got[:accepted + 1]]  # the accepted guesses are the model's own picks; plus one more
            out.extend(new)
            cur, pos = new[-1], pos + accepted + 1
        return out[:n], passes

    def decode(self, first_token: int, start_pos: int, n: int):
        """Resident greedy decode of n tokens -> (tokens int32[n], device milliseconds)."""
        out = np.zeros(n, dtype=np.int32)
        ms = C.c_float(0)
        rc = self._L.llamd_model_decode(self._h, int(first_token), int(start_pos), int(n), out.ctypes.data_as(C.c_void_p), C.byref(ms))
        if rc != 0:
            raise backend.Other("decode: " + self._err())
        return out, float(ms.value)

    def bench_matvecs(self, iters: int, nseq: int = 1):
        """-> (device ms for iters passes of the matvec launches only, launches per pass)"""
        ms, n = C.c_float(0), C.c_int(0)
        if self._L.llamd_model_bench_matvecs(self._h, iters, nseq, C.byref(ms), C.byref(n)) != 0:
            raise backend.Other("bench_matvecs: " + self._err())
        return float(ms.value), int(n.value)

    def launches_per_pass(self) -> int:
        return int(self._L.llamd_model_launches_per_pass(self._h))

    PHASES = ("embed", "attn_norm", "qkv", "rope", "attention", "quant", "attn_out", "ffn_norm", "router", "gate_up", "silu", "down",
              "lm_head", "argmax")

    def profile_pass(self, token: int, pos: int) -> dict:
        """Per-phase milliseconds of one un-graphed pass (summed over layers). A diagnostic, not a throughput."""
        ms = np.zeros(len(self.PHASES), dtype=np.float32)
        if self._L.llamd_model_profile_pass(self._h, int(token), int(pos), ms.ctypes.data_as(C.c_void_p)) != 0:
            raise backend.Other("profile_pass: " + self._err())
        return dict(zip(self.PHASES, ms.tolist()))

    def logits(self, nseq: int = 1) -> np.ndarray:
        out = np.zeros((nseq, self.hp["n_vocab"]), dtype=np.float32)
        if self._L.llamd_model_logits(self._h, out.ctypes.data_as(C.c_void_p), nseq) != 0:
            raise backend.Other("logits: " + self._err())
        return out

    def read_trace(self):
        """-> (x [n_layer][max_seq][n_embd], ids [n_layer][max_seq][n_used]) of the last traced pass"""
        hp = self.hp
        x = np.zeros((hp["n_layer"], self.max_seq, hp["n_embd"]), dtype=np.float32)
        ids = np.zeros((hp["n_layer"], self.max_seq, hp["n_expert_used"]), dtype=np.int32)
        if self._L.llamd_model_read_trace(self._h, x.ctypes.data_as(C.c_void_p), ids.ctypes.data_as(C.c_void_p)) != 0:
            raise backend.Other("read_trace: tracing is off")
        return x, ids

    def read_kv(self, layer: int, n_pos: int, seq: int = 0):
        kvd = self.hp["n_head_kv"] * self.hp["head_dim"]
        k = np.zeros(n_pos * kvd, dtype=np.float32)
        v = np.zeros(n_pos * kvd, dtype=np.float32)
        if self._L.llamd_model_read_kv(self._h, layer, seq, n_pos, k.ctypes.data_as(C.c_void_p), v.ctypes.data_as(C.c_void_p)) != 0:
            raise backend.Malformed("read_kv: out of range")
        return k, v

    def weight_bytes(self) -> int:
        return int(self._L.llamd_model_weight_bytes(self._h))

    def hparams(self) -> dict:
        return dict(self.hp)

    def free(self) -> None:
        if getattr(self, "_h", None):
            self._L.llamd_model_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

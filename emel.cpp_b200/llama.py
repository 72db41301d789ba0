"""Decoder-session bindings (include/emelb_llama.h): a Llama-architecture decode
loop that stays on the device, mirroring the reference generator's run_decode
(src/emel/text/generator/detail.hpp:4860-4914)."""
from __future__ import annotations

import ctypes as C

import numpy as np

import emel_cpp_b200 as eb

_P = C.c_void_p

# tensor roles (include/emelb_llama.h)
TOKEN_EMBD, OUTPUT_NORM, OUTPUT, ATTN_NORM, ATTN_Q, ATTN_K, ATTN_V, ATTN_OUT, FFN_NORM, FFN_GATE, FFN_UP, FFN_DOWN = range(12)
LAYER_ROLES = (ATTN_NORM, ATTN_Q, ATTN_K, ATTN_V, ATTN_OUT, FFN_NORM, FFN_GATE, FFN_UP, FFN_DOWN)


class Config(C.Structure):
    _fields_ = [("n_layer", C.c_int32), ("n_embd", C.c_int32), ("n_head", C.c_int32), ("n_head_kv", C.c_int32),
                ("head_dim", C.c_int32), ("n_ff", C.c_int32), ("n_vocab", C.c_int32), ("n_ctx", C.c_int32),
                ("rope_dim", C.c_int32), ("rope_neox", C.c_int32), ("rope_freq_base", C.c_float), ("rms_eps", C.c_float),
                ("kv_block", C.c_int32), ("shard_rank", C.c_int32), ("shard_count", C.c_int32)]


SIGNATURES = {
    "emelb_llama_check_config": [C.POINTER(Config)],
    "emelb_llama_create": [_P, C.POINTER(Config), C.POINTER(_P)],
    "emelb_llama_destroy": [_P],
    "emelb_llama_bind": [_P, C.c_int32, C.c_int32, C.POINTER(eb.View)],
    "emelb_llama_decode": [_P, C.c_int32, C.c_int32, _P, C.POINTER(C.c_int32)],
    "emelb_llama_prefill": [_P, C.POINTER(C.c_int32), C.c_int32, C.c_int32],
    "emelb_llama_generate": [_P, C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_int32)],
    "emelb_llama_launches_per_token": [_P, C.POINTER(C.c_int32)],
    "emelb_llama_set_step_mode": [_P, C.c_int32],
    "emelb_llama_set_prefill_batch": [_P, C.c_int32],
    "emelb_llama_set_join_fusion": [_P, C.c_int32],
    "emelb_llama_set_sequences": [_P, C.c_int32],
    "emelb_llama_select_sequence": [_P, C.c_int32],
    "emelb_llama_decode_batch": [_P, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.c_int32, _P, C.POINTER(C.c_int32)],
    "emelb_llama_generate_batch": [_P, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.c_int32, C.c_int32, C.POINTER(C.c_int32)],
    "emelb_llama_batch_launches_per_step": [_P, C.POINTER(C.c_int32)],
    "emelb_llama_decode_profile": [_P, C.c_int32, C.c_int32, _P, C.c_uint64],
    "emelb_llama_exchange_export": [_P, _P, C.c_uint64],
    "emelb_llama_exchange_attach": [_P, _P, C.c_uint64],
    "emelb_llama_exchange_detach": [_P],
}


EXCHANGE_HANDLE_BYTES = 64


def register(lib):
    for name, args in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = C.c_uint32
        fn.argtypes = args


def config(n_layer, n_embd, n_head, n_head_kv, head_dim, n_ff, n_vocab, n_ctx, rope_freq_base=500000.0, rms_eps=1e-5,
           rope_dim=None, rope_neox=0, kv_block=16, shard_rank=0, shard_count=1) -> Config:
    return Config(n_layer, n_embd, n_head, n_head_kv, head_dim, n_ff, n_vocab, n_ctx,
                  head_dim if rope_dim is None else rope_dim, rope_neox, rope_freq_base, rms_eps, kv_block,
                  shard_rank, shard_count)


def check_config(cfg: Config) -> int:
    """emelb_llama_check_config: the error bitmask for a configuration, without a device."""
    return int(eb.lib().emelb_llama_check_config(C.byref(cfg)))


def matrix_shapes(cfg: Config):
    """role -> (K, M) of each matrix, as emelb_llama_bind checks them.  In a row-sharded session
    (shard_count G > 1) M is this rank's interval: M/G rows, all K columns; the embedding table is whole."""
    qd, kvd, g = cfg.n_head * cfg.head_dim, cfg.n_head_kv * cfg.head_dim, max(1, cfg.shard_count)
    return {TOKEN_EMBD: (cfg.n_embd, cfg.n_vocab), OUTPUT: (cfg.n_embd, cfg.n_vocab // g),
            ATTN_Q: (cfg.n_embd, qd // g), ATTN_K: (cfg.n_embd, kvd // g), ATTN_V: (cfg.n_embd, kvd // g),
            ATTN_OUT: (qd, cfg.n_embd // g), FFN_GATE: (cfg.n_embd, cfg.n_ff // g), FFN_UP: (cfg.n_embd, cfg.n_ff // g),
            FFN_DOWN: (cfg.n_ff, cfg.n_embd // g)}


def shard_rows(m: int, rank: int, count: int):
    """(first row, row count) of rank's interval of an M-row matrix: equal contiguous intervals, the split
    the reference's fixed row slices make when M divides evenly (src/emel/kernel/matmul/actions.hpp:49-66)."""
    if count < 1 or not 0 <= rank < count or m % count != 0:
        raise ValueError(f"{m} rows do not split evenly over {count} ranks")
    return rank * (m // count), m // count


def merge_argmax_pairs(pairs):
    """Host mirror of the sharded greedy head's last step: from each rank's (value, global row)
    candidate, the highest value and on ties the lowest row (src/emel/kernel/detail.hpp:3720-3723)."""
    best_v, best_r = pairs[0]
    for v, r in pairs[1:]:
        if v > best_v or (v == best_v and r < best_r):
            best_v, best_r = v, r
    return best_r


class Session:
    def __init__(self, backend: eb.Backend, cfg: Config):
        self.be, self.cfg = backend, cfg
        self._h = _P()
        err = eb.lib().emelb_llama_create(backend.handle, C.byref(cfg), C.byref(self._h))
        if err != eb.OK:
            raise eb.BackendError(f"emelb_llama_create failed with error mask {err}")
        self.last_error = eb.OK

    def close(self):
        if self._h:
            eb.lib().emelb_llama_destroy(self._h)
            self._h = _P()

    def _ret(self, err):
        self.last_error = err
        return err == eb.OK

    def bind_matrix(self, layer: int, role: int, data, t: int) -> bool:
        k, m = matrix_shapes(self.cfg)[role]
        if t in (eb.F32, eb.F16):
            v = eb.dense_view(data, t, [k, m])
        else:
            v = eb.quant_view(data, t, k, m)
        return self._ret(eb.lib().emelb_llama_bind(self._h, layer, role, C.byref(v)))

    def bind_norm(self, layer: int, role: int, data) -> bool:
        v = eb.dense_view(data, eb.F32, [self.cfg.n_embd, 1])
        return self._ret(eb.lib().emelb_llama_bind(self._h, layer, role, C.byref(v)))

    def decode(self, token: int, position: int, want_logits: bool = False):
        """-> next token id (greedy) or, with want_logits, the f32 logits."""
        if want_logits:
            logits = np.zeros(self.cfg.n_vocab, np.float32)
            if not self._ret(eb.lib().emelb_llama_decode(self._h, token, position, logits.ctypes.data, None)):
                raise eb.BackendError(f"decode failed with error mask {self.last_error}")
            return logits
        out = C.c_int32(-1)
        if not self._ret(eb.lib().emelb_llama_decode(self._h, token, position, None, C.byref(out))):
            raise eb.BackendError(f"decode failed with error mask {self.last_error}")
        return out.value

    def prefill(self, tokens, start_pos: int = 0) -> bool:
        arr = np.ascontiguousarray(tokens, np.int32)
        return self._ret(eb.lib().emelb_llama_prefill(self._h, arr.ctypes.data_as(C.POINTER(C.c_int32)), arr.size, start_pos))

    def generate(self, first_token: int, start_pos: int, n: int):
        out = np.zeros(n, np.int32)
        if not self._ret(eb.lib().emelb_llama_generate(self._h, first_token, start_pos, n,
                                                       out.ctypes.data_as(C.POINTER(C.c_int32)))):
            raise eb.BackendError(f"generate failed with error mask {self.last_error}")
        return out

    def exchange_export(self) -> bytes:
        """Handle of this rank's exchange arena (sharded sessions), to be all-gathered by the caller."""
        buf = (C.c_uint8 * EXCHANGE_HANDLE_BYTES)()
        if not self._ret(eb.lib().emelb_llama_exchange_export(self._h, C.addressof(buf), EXCHANGE_HANDLE_BYTES)):
            raise eb.BackendError(f"exchange_export failed with error mask {self.last_error}")
        return bytes(buf)

    def exchange_attach(self, handles) -> bool:
        """handles: every rank's exchange_export() in rank order; switches the joins to peer stores."""
        blob = b"".join(handles)
        buf = (C.c_uint8 * len(blob)).from_buffer_copy(blob)
        return self._ret(eb.lib().emelb_llama_exchange_attach(self._h, C.addressof(buf), len(blob)))

    def exchange_detach(self) -> bool:
        """Unmap the peers' arenas; call on every rank, synchronise the ranks, then close()."""
        return self._ret(eb.lib().emelb_llama_exchange_detach(self._h))

    def launches_per_token(self) -> int:
        v = C.c_int32(0)
        eb.lib().emelb_llama_launches_per_token(self._h, C.byref(v))
        return v.value

    def set_prefill_batch(self, max_tokens: int) -> bool:
        """Prompt tokens per batch of prefill(): 0 walks the prompt token by token."""
        return self._ret(eb.lib().emelb_llama_set_prefill_batch(self._h, max_tokens))

    def set_sequences(self, n_seq: int) -> bool:
        """Hold n_seq KV caches (reallocated and cleared); decode_batch / generate_batch step sequences 0..n-1 together."""
        return self._ret(eb.lib().emelb_llama_set_sequences(self._h, n_seq))

    def select_sequence(self, seq: int) -> bool:
        """The sequence prefill / decode / generate work on."""
        return self._ret(eb.lib().emelb_llama_select_sequence(self._h, seq))

    def decode_batch(self, tokens, positions, want_logits: bool = False):
        """One step of len(tokens) sequences -> next ids, or with want_logits (ids, logits [n_seq, n_vocab])."""
        t = np.ascontiguousarray(tokens, np.int32)
        p = np.ascontiguousarray(positions, np.int32)
        out = np.zeros(t.size, np.int32)
        logits = np.zeros((self.cfg.n_vocab, t.size), np.float32) if want_logits else None
        ip = C.POINTER(C.c_int32)
        if not self._ret(eb.lib().emelb_llama_decode_batch(self._h, t.ctypes.data_as(ip), p.ctypes.data_as(ip), t.size,
                                                           logits.ctypes.data if want_logits else None, out.ctypes.data_as(ip))):
            raise eb.BackendError(f"decode_batch failed with error mask {self.last_error}")
        return (out, logits.T.copy()) if want_logits else out

    def generate_batch(self, first_tokens, start_positions, n_steps: int):
        """n_steps greedy steps of len(first_tokens) sequences fed back on the device -> ids [n_steps, n_seq]."""
        t = np.ascontiguousarray(first_tokens, np.int32)
        p = np.ascontiguousarray(start_positions, np.int32)
        out = np.zeros((n_steps, t.size), np.int32)
        ip = C.POINTER(C.c_int32)
        if not self._ret(eb.lib().emelb_llama_generate_batch(self._h, t.ctypes.data_as(ip), p.ctypes.data_as(ip), t.size, n_steps,
                                                             out.ctypes.data_as(ip))):
            raise eb.BackendError(f"generate_batch failed with error mask {self.last_error}")
        return out

    def batch_launches_per_step(self) -> int:
        v = C.c_int32(0)
        eb.lib().emelb_llama_batch_launches_per_step(self._h, C.byref(v))
        return v.value

    def set_join_fusion(self, on: bool) -> bool:
        """Sharded sessions with peers attached: joins inside the neighbouring kernels (default) or one join kernel each."""
        return self._ret(eb.lib().emelb_llama_set_join_fusion(self._h, 1 if on else 0))

    def set_window(self, window) -> bool:
        """Attach a bound, streaming LayerWindow (or None to detach): layer tensors bound afterwards by an address
        inside its source are read from the window's slots (emelb_llama_set_window)."""
        self._window = window   # kept alive with the session
        return self._ret(eb.lib().emelb_llama_set_window(self._h, window.handle if window is not None else None))

    def set_step_mode(self, mode: int) -> bool:
        """0: the chain of per-operation launches (default); 1: one persistent kernel per token where the session qualifies."""
        return self._ret(eb.lib().emelb_llama_set_step_mode(self._h, mode))

    def decode_profile(self, token: int, position: int):
        """-> (n_layer, 16) nanosecond stamps of the one-kernel step (see emelb_llama_decode_profile)."""
        out = np.zeros((self.cfg.n_layer, 16), np.uint64)
        if not self._ret(eb.lib().emelb_llama_decode_profile(self._h, token, position, out.ctypes.data, out.size)):
            raise eb.BackendError(f"decode_profile failed with error mask {self.last_error}")
        return out

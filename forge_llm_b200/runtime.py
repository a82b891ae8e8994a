"""Host-side mirror of the generated ``model::`` surface on top of the C ABI.

Names and argument meaning follow the reference's generated module
(crates/forgellm-codegen-cpu/src/emit.rs): ``Weights``/``KVCache`` become :class:`Model` and
:class:`KVCache`; ``forward(token, &weights, &mut cache)`` (emit.rs:4029) and
``forward_prefill(tokens, &weights, &mut cache)`` (emit.rs:4553) become methods of the model.
Errors the reference raises as panics (cache overrun, bad slice lengths) surface as
:class:`ForgeError`.  All buffers crossing this layer are numpy arrays in host memory; the
library copies to and from the GPU itself.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import ForgeError, ForgeModelConfig, check, lib


def _cfg_struct(c: dict, tp_rank: int = 0, tp_world: int = 1) -> ForgeModelConfig:
    return ForgeModelConfig(c["hidden_size"], c["intermediate_size"], c["num_layers"], c["num_heads"],
                            c["num_kv_heads"], c["head_dim"], c["vocab_size"], c["max_seq_len"],
                            c["rms_norm_eps"], c["rope_theta"], c["quant"], int(c.get("qkv_bias", 0)),
                            tp_rank, tp_world, int(c.get("sliding_window", 0) or 0),
                            (C.c_int32 * 8)(*[int(v) for v in (c.get("proj_quant") or [0] * 8)]))


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def weights_bin_size(c: dict) -> int:
    s = _cfg_struct(c)
    return int(lib.forge_weights_bin_size(C.byref(s)))


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    """Host quantiser of the exporter (weight_loader.rs:1454-1486)."""
    x = np.ascontiguousarray(x, np.float32).ravel()
    out = np.empty(x.size // 32 * 34, np.uint8)
    check(lib.forge_quantize_q8_0_host(_p(x), x.size, _p(out)))
    return out


def quantize_q4_0(x: np.ndarray, signed_max: bool = True) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32).ravel()
    out = np.empty(x.size // 32 * 18, np.uint8)
    check(lib.forge_quantize_q4_0_host(_p(x), x.size, _p(out), int(signed_max)))
    return out


def quantize_kquant(quant: int, x: np.ndarray) -> np.ndarray:
    """f32 -> Q4_K (quant 12) or Q6_K (quant 14) super-blocks with the exporter's host quantisers."""
    x = np.ascontiguousarray(x, np.float32).ravel()
    out = np.empty(x.size // 256 * (144 if quant == 12 else 210), np.uint8)
    check((lib.forge_quantize_q4_k_host if quant == 12 else lib.forge_quantize_q6_k_host)(_p(x), x.size, _p(out)))
    return out


class KVCache:
    """``KVCache`` of the generated module (emit.rs:3954-4015): fp16, paged, ``batch`` sequences."""

    def __init__(self, model: "Model", max_seq: int | None = None, batch: int = 1):
        self.model = model
        self.batch = batch
        h = C.c_void_p()
        check(lib.forge_kv_create(model._h, int(max_seq or model.cfg["max_seq_len"]), batch, C.byref(h)))
        self._h = h

    def reset(self) -> None:
        check(lib.forge_kv_reset(self._h))

    def len(self, seq: int = 0) -> int:
        return int(lib.forge_kv_len(self._h, seq))

    def read(self, layer: int, which: int, seq: int = 0) -> np.ndarray:
        kvd = self.model.cfg["num_kv_heads"] * self.model.cfg["head_dim"] // self.model.tp_world
        out = np.empty((self.len(seq), kvd), np.float32)
        check(lib.forge_kv_read(self._h, seq, layer, which, _p(out)))
        return out

    def save(self, seq: int = 0) -> np.ndarray:
        """The sequence's cache as a byte image (fp16 rows behind a small header)."""
        out = np.empty(int(lib.forge_kv_save_size(self._h, seq)), np.uint8)
        check(lib.forge_kv_save(self._h, seq, _p(out), out.size))
        return out

    def load(self, data, seq: int = 0) -> None:
        """Restores a saved sequence; also takes the reference's int8 cache file (converted to fp16)."""
        buf = np.ascontiguousarray(np.frombuffer(data, np.uint8) if not isinstance(data, np.ndarray) else data, np.uint8)
        check(lib.forge_kv_load(self._h, seq, _p(buf), buf.size))

    def close(self) -> None:
        if getattr(self, "_h", None):
            lib.forge_kv_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


TP_ID_BYTES = 128  # FORGE_TP_ID_BYTES
TP_HANDLE_BYTES = 64  # FORGE_TP_HANDLE_BYTES


class Model:
    """``Weights`` + ``forward`` / ``forward_prefill`` of the generated module."""

    def __init__(self, cfg: dict, weights_bin: np.ndarray, device: int = 0, tp_rank: int = 0, tp_world: int = 1):
        self.cfg = dict(cfg)
        self.tp_world = tp_world
        blob = np.ascontiguousarray(weights_bin, np.uint8)
        s = _cfg_struct(cfg, tp_rank, tp_world)
        h = C.c_void_p()
        check(lib.forge_model_create(C.byref(s), _p(blob), blob.size, device, C.byref(h)))
        self._h = h
        self.device = device

    @property
    def stream(self) -> int:
        return int(lib.forge_model_stream(self._h) or 0)

    @staticmethod
    def tp_unique_id() -> np.ndarray:
        """Rendezvous id for the tensor-parallel ranks (rank 0 creates it, the others receive it)."""
        out = np.zeros(TP_ID_BYTES, np.uint8)
        check(lib.forge_tp_unique_id(_p(out)))
        return out

    def tp_init(self, unique_id: np.ndarray) -> None:
        """Joins the tensor-parallel group (collective over all ``tp_world`` ranks)."""
        uid = np.ascontiguousarray(unique_id, np.uint8)
        if uid.size != TP_ID_BYTES:
            raise ValueError(f"the rendezvous id is {TP_ID_BYTES} bytes")
        check(lib.forge_model_tp_init(self._h, _p(uid)))

    def tp_exchange_handle(self) -> np.ndarray:
        """This rank's handle to its peer-memory exchange buffer (to be gathered over all ranks, in rank order)."""
        out = np.zeros(TP_HANDLE_BYTES, np.uint8)
        check(lib.forge_model_tp_exchange_export(self._h, _p(out)))
        return out

    def tp_exchange_attach(self, handles: np.ndarray) -> None:
        """Maps the peers' exchange buffers; the batch-1 decode step then sums over peer memory."""
        h = np.ascontiguousarray(handles, np.uint8).reshape(-1)
        if h.size != TP_HANDLE_BYTES * self.tp_world:
            raise ValueError("one handle per rank, in rank order")
        check(lib.forge_model_tp_exchange_attach(self._h, _p(h)))

    def new_cache(self, max_seq: int | None = None, batch: int = 1) -> KVCache:
        return KVCache(self, max_seq, batch)

    def forward(self, token: int, cache: KVCache, seq: int = 0, want_logits: bool = True):
        logits = np.empty(self.cfg["vocab_size"], np.float32) if want_logits else None
        check(lib.forge_forward_seq(self._h, cache._h, seq, int(token), _p(logits)))
        return logits

    def forward_prefill(self, tokens, cache: KVCache, seq: int = 0, want_logits: bool = True):
        t = np.ascontiguousarray(tokens, np.uint32)
        logits = np.empty(self.cfg["vocab_size"], np.float32) if want_logits else None
        check(lib.forge_forward_prefill_seq(self._h, cache._h, seq, _p(t), t.size, _p(logits)))
        return logits

    def forward_batch(self, tokens, cache: KVCache, want_logits: bool = True):
        t = np.ascontiguousarray(tokens, np.uint32)
        logits = np.empty((t.size, self.cfg["vocab_size"]), np.float32) if want_logits else None
        check(lib.forge_forward_batch(self._h, cache._h, t.size, _p(t), _p(logits)))
        return logits

    def generate_greedy(self, prompt, n_new: int, cache: KVCache) -> np.ndarray:
        """Prefill + ``n_new`` greedy steps with token selection on the device (project.rs:714-751
        at temperature 0, repeat penalty 1.0).  Host prompt in, host token ids out."""
        t = np.ascontiguousarray(prompt, np.uint32)
        out = np.empty(n_new, np.uint32)
        check(lib.forge_generate_greedy(self._h, cache._h, _p(t), t.size, n_new, _p(out)))
        return out

    def decode_greedy_batch(self, first_tokens, n_new: int, cache: KVCache) -> np.ndarray:
        t = np.ascontiguousarray(first_tokens, np.uint32)
        out = np.empty((n_new, t.size), np.uint32)
        check(lib.forge_decode_greedy_batch(self._h, cache._h, t.size, _p(t), n_new, _p(out)))
        return out

    def set_gemm_passes(self, passes: int) -> None:
        """3 = split-precision prefill GEMMs (default), 1 = a single fp16 tensor-core pass."""
        check(lib.forge_model_set_gemm_passes(self._h, passes))

    def set_prefill_mode(self, mode: int) -> None:
        """K-quant models: 0 = prompt token by token (default, the reference's structure), 1 = batched GEMMs."""
        check(lib.forge_model_set_prefill_mode(self._h, mode))

    def set_wait_limit(self, polls: int) -> None:
        """Polls a device-side wait makes before it gives up (the call then fails with status TIMEOUT)."""
        check(lib.forge_model_set_wait_limit(self._h, polls))

    def trace(self, enable: bool) -> None:
        check(lib.forge_hidden_trace_enable(self._h, int(enable)))

    def read_trace(self, rows: int) -> np.ndarray:
        out = np.empty((self.cfg["num_layers"], rows, self.cfg["hidden_size"]), np.float32)
        got = C.c_int32()
        check(lib.forge_hidden_trace_read(self._h, _p(out), out.size, C.byref(got)))
        if got.value != rows:
            raise ForgeError(1, f"trace holds {got.value} rows, asked for {rows}")
        return out

    def score_corpus(self, tokens, cache: "KVCache", chunk_size: int = 512, max_chunks: int = 0):
        """Token-by-token perplexity like the generated binary's --score-corpus: (mean NLL in nats, perplexity, count)."""
        t = np.ascontiguousarray(tokens, np.uint32)
        total, count, chunks = 0.0, 0, 0
        for start in range(0, t.size, chunk_size):
            if max_chunks and chunks >= max_chunks:
                break
            chunk = t[start:start + chunk_size]
            chunks += 1
            if chunk.size < 2:
                continue
            nll = np.empty(chunk.size - 1, np.float64)
            check(lib.forge_score_chunk(self._h, cache._h, _p(chunk), chunk.size, _p(nll)))
            for v in nll:  # sequential f64 sum, as the reference accumulates
                total += float(v)
            count += nll.size
        mean = total / max(count, 1)
        return mean, float(np.exp(mean)), count

    def last_timing(self):
        a, b, n = C.c_float(), C.c_float(), C.c_int64()
        check(lib.forge_last_timing(self._h, C.byref(a), C.byref(b), C.byref(n)))
        return a.value, b.value, n.value

    def close(self) -> None:
        if getattr(self, "_h", None):
            lib.forge_model_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

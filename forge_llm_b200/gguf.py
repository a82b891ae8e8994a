"""GGUF checkpoints as input: configuration and ``weights.bin`` image through the library's reader.

    g = GgufFile(open("model.gguf", "rb").read())      # or a numpy memmap
    model = runtime.Model(g.config(), g.weights_bin())

Mirrors ``forge export-weights`` of the reference (crates/forgellm-cli/src/main.rs:2506-2757).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import ForgeModelConfig, check, lib


class GgufFile:
    def __init__(self, data):
        self._h = None
        self._buf = np.frombuffer(data, np.uint8) if not isinstance(data, np.ndarray) else np.ascontiguousarray(data, np.uint8)
        h = C.c_void_p()
        check(lib.forge_gguf_open(self._buf.ctypes.data_as(C.c_void_p), self._buf.size, C.byref(h)))
        self._h = h

    def close(self) -> None:
        if self._h:
            lib.forge_gguf_close(self._h)
            self._h = None

    def __del__(self):
        self.close()

    @property
    def version(self) -> int:
        return int(lib.forge_gguf_version(self._h))

    @property
    def data_offset(self) -> int:
        return int(lib.forge_gguf_data_offset(self._h))

    def tensors(self) -> list[dict]:
        out = []
        for i in range(int(lib.forge_gguf_tensor_count(self._h))):
            name, typ, nd = C.c_char_p(), C.c_int32(), C.c_int32()
            dims = (C.c_uint64 * 4)()
            off, size = C.c_uint64(), C.c_uint64()
            check(lib.forge_gguf_tensor_info(self._h, i, C.byref(name), C.byref(typ), C.byref(nd), dims, C.byref(off), C.byref(size)))
            out.append({"name": name.value.decode(), "type": typ.value, "dims": [int(dims[d]) for d in range(nd.value)],
                        "offset": int(off.value), "size": int(size.value)})
        return out

    def tensor_f32(self, index: int) -> np.ndarray:
        """Tensor ``index`` dequantised to f32 (flat)."""
        t = self.tensors()[index]
        n = int(np.prod(t["dims"])) if t["dims"] else 1
        out = np.empty(n, np.float32)
        check(lib.forge_gguf_tensor_to_f32(self._h, index, out.ctypes.data_as(C.c_void_p), n))
        return out

    def config(self) -> dict:
        c = ForgeModelConfig()
        check(lib.forge_gguf_model_config(self._h, C.byref(c)))
        return {"hidden_size": c.hidden_size, "intermediate_size": c.intermediate_size, "num_layers": c.num_layers,
                "num_heads": c.num_heads, "num_kv_heads": c.num_kv_heads, "head_dim": c.head_dim, "vocab_size": c.vocab_size,
                "max_seq_len": c.max_seq_len, "rms_norm_eps": c.rms_norm_eps, "rope_theta": c.rope_theta, "quant": c.quant,
                "qkv_bias": c.qkv_bias, "sliding_window": c.sliding_window, "name": "gguf",
                "proj_quant": [int(v) for v in c.proj_quant]}

    def weights_bin(self) -> np.ndarray:
        n = int(lib.forge_gguf_weights_bin_size(self._h))
        if n == 0:
            check(lib.forge_gguf_export_weights_bin(self._h, None, 0))  # raises with the library's message
        out = np.empty(n, np.uint8)
        check(lib.forge_gguf_export_weights_bin(self._h, out.ctypes.data_as(C.c_void_p), n))
        return out

"""CPU-side checks: the C-ABI library loads and exports what the header declares, the host
quantisers and the synthetic-weights writer agree with the oracle, errors are reported as
status codes (no compute call needs a GPU here)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "forge_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(forge_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from forge_llm_b200 import _lib
    names = _declared_symbols()
    assert len(names) >= 30
    for n in names:
        assert hasattr(_lib.lib, n), f"{n} declared in forge_b200.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), set(names) ^ set(_lib.SIGNATURES)


def test_no_torch_types_in_header():
    text = open(os.path.join(ROOT, "include", "forge_b200.h")).read()
    assert "torch" not in text.lower().replace("no torch types", "") and "at::" not in text


def test_product_never_touches_the_oracle():
    # the shipped package and the CUDA sources must not import, link or execute oracle/
    pkg = os.path.join(ROOT, "forge_llm_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                assert "oracle" not in open(os.path.join(dirpath, f)).read().lower(), f


def test_weights_bin_size_agrees(oracle):
    from forge_llm_b200 import configs, runtime, synth
    mixed = [configs.tiny(12, ffn=512), configs.with_proj_quant(configs.tiny(12, ffn=512, bias=1), v=14, down=14, lm_head=14),
             configs.with_proj_quant(configs.tiny(4), lm_head=8)]
    for c in list(configs.CONFIGS.values()) + [configs.tiny(4, bias=1)] + mixed:
        oc = oracle.make_config(c)
        assert runtime.weights_bin_size(c) == synth.weights_bin_size(c) == oracle.lib().fo_weights_bin_size(C.byref(oc))


def test_host_quantisers_match_oracle_bit_for_bit(oracle):
    from forge_llm_b200 import runtime, synth
    rng = np.random.default_rng(7)
    x = rng.standard_normal(32 * 2048, dtype=np.float32) * 0.02
    x[:32] = 0.0
    x[64] = 3.0
    q8 = oracle.quantize_q8_0(x)
    assert np.array_equal(runtime.quantize_q8_0(x), q8) and np.array_equal(synth.quantize_q8_0(x), q8)
    q4 = oracle.quantize_q4_0(x, "signed")
    assert np.array_equal(runtime.quantize_q4_0(x, True), q4) and np.array_equal(synth.quantize_q4_0(x), q4)
    assert np.array_equal(runtime.quantize_q4_0(x, False), oracle.quantize_q4_0(x, "ref"))
    assert np.array_equal(synth.dequantize(8, q8, x.size), oracle.dequant_q8_0(q8, x.size))
    assert np.array_equal(synth.dequantize(4, q4, x.size), oracle.dequant_q4_0(q4, x.size))


def test_host_kquant_quantisers_match_oracle_bit_for_bit(oracle):
    from forge_llm_b200 import runtime
    rng = np.random.default_rng(9)
    n = 256 * 48
    cases = [rng.standard_normal(n).astype(np.float32) * 0.05, np.zeros(n, np.float32), np.full(n, 0.3, np.float32),
             (np.abs(rng.standard_normal(n)) + 1).astype(np.float32), ((np.arange(n) - n / 2) * 0.005).astype(np.float32)]
    spiky = rng.standard_normal(n).astype(np.float32) * 0.02
    spiky[::97] *= 30
    for x in cases + [spiky]:
        for q in (12, 14):
            assert np.array_equal(runtime.quantize_kquant(q, x), oracle.quantize_kquant(q, x))


def test_rope_table_matches_oracle(oracle):
    from forge_llm_b200._lib import lib
    for hd, theta in ((64, 1e5), (96, 1e4), (128, 5e5)):
        tab = np.empty((300, hd // 2, 2), np.float32)
        assert lib.forge_rope_table(tab.ctypes.data_as(C.c_void_p), 300, hd, theta) == 0
        f = oracle.rope_freqs(hd, theta)
        x = np.zeros(hd, np.float32)
        x[0::2] = 1.0  # (1, 0) pairs rotate to (cos, sin)
        for pos in (0, 1, 17, 299):
            y = oracle.rope(x, pos, hd, 1, f)
            assert np.array_equal(y[0::2], tab[pos, :, 0]) and np.array_equal(y[1::2], tab[pos, :, 1])


def test_synthetic_model_layout_and_tied_embedding(oracle):
    from forge_llm_b200 import configs, synth
    c = configs.tiny(8)
    c["tied"] = True
    blob = synth.make_weights_bin(c)
    assert blob.size == synth.weights_bin_size(c)
    V, h = c["vocab_size"], c["hidden_size"]
    emb = blob[:V * h * 4].view(np.float32)
    lm = blob[-V * (h // 32) * 34:]
    assert np.array_equal(emb, oracle.dequant_q8_0(lm, V * h))
    assert np.array_equal(blob, synth.make_weights_bin(c))  # deterministic
    m = oracle.OracleModel(c, blob)
    assert np.isfinite(m.forward_prefill(synth.prompt_tokens(c, 12))).all()
    with pytest.raises(ValueError):
        oracle.OracleModel(c, blob[:-1])


def test_errors_are_status_codes_not_aborts():
    from forge_llm_b200 import configs, runtime, synth
    from forge_llm_b200._lib import ForgeError, lib
    c = configs.tiny(8)
    blob = synth.make_weights_bin(c)
    bad = dict(c, head_dim=80)
    with pytest.raises(ForgeError) as e:
        runtime.Model(bad, blob)
    assert e.value.code == 2  # FORGE_ERR_SHAPE
    with pytest.raises(ForgeError) as e:
        runtime.Model(dict(c, quant=5), blob)
    assert e.value.code == 1
    if lib.forge_device_count() == 0:
        with pytest.raises(ForgeError) as e:
            runtime.Model(c, blob)
        assert e.value.code == 4 and "no CPU fallback" in str(e.value)
        assert lib.forge_rms_norm(None, None, None, 1, 4, C.c_float(1e-5), None) == 4
    else:
        with pytest.raises(ForgeError) as e:
            runtime.Model(c, blob[:-2])
        assert e.value.code == 2


def test_algorithmic_work_tables():
    # per-token decode bytes and prefill flops used for the rooflines
    from forge_llm_b200 import configs
    c1, c2 = configs.CONFIGS["c1"], configs.CONFIGS["c2"]
    assert configs.weight_elems(c1) == 134_479_872
    assert configs.weight_elems(c2) == 1_235_746_816
    assert abs(configs.decode_bytes_per_token(c2, 1565) / 1e6 - 746.4) < 0.5
    assert abs(configs.prefill_flops(c2, 1501) / 1e12 - 3.07) < 0.05

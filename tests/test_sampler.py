"""Token selection and generation loop of the generated main.rs (project.rs:501-551, :714-751), host code of the library.

The checker is a direct Python restatement with float32 scalars, libm's expf and sequential sums; the reference holds no
numeric test for this sampler, so the restatement is pinned only by reading (inputs avoid exactly equal probabilities,
where the reference's sort_unstable_by leaves the order open)."""
import ctypes as C

import numpy as np
import pytest

from forge_llm_b200._lib import ForgeSampling, check, lib

_libm = C.CDLL("libm.so.6")
_libm.expf.restype = C.c_float
_libm.expf.argtypes = [C.c_float]
F = np.float32


def ref_repeat_penalty(logits, recent, penalty):
    if penalty <= 1.0:
        return
    for tok in recent:
        if tok < len(logits):
            logits[tok] = logits[tok] / F(penalty) if logits[tok] > 0 else logits[tok] * F(penalty)


def ref_sample(logits, temperature, top_k, top_p, state):
    n = len(logits)
    if temperature <= 0.0:
        return int(np.flatnonzero(logits == logits.max())[-1]), state
    for i in range(n):
        logits[i] = logits[i] / F(temperature)
    mx = F(-np.inf)
    for i in range(n):
        mx = max(mx, logits[i])
    s = F(0)
    for i in range(n):
        logits[i] = F(_libm.expf(float(logits[i] - mx)))
        s = F(s + logits[i])
    for i in range(n):
        logits[i] = logits[i] / s
    order = sorted(range(n), key=lambda i: -float(logits[i]))
    if 0 < top_k < n:
        for i in order[top_k:]:
            logits[i] = F(0)
    if 0.0 < top_p < 1.0:
        c = F(0)
        for i in order:
            c = F(c + logits[i])
            if c > F(top_p):
                logits[i] = F(0)
    s = F(0)
    for i in range(n):
        s = F(s + logits[i])
    if s > 0:
        for i in range(n):
            logits[i] = logits[i] / s
    state ^= (state << 13) & 0xFFFFFFFFFFFFFFFF
    state ^= state >> 7
    state ^= (state << 17) & 0xFFFFFFFFFFFFFFFF
    r = F(F(state) / F(18446744073709551616.0))
    c = F(0)
    for i in range(n):
        c = F(c + logits[i])
        if c >= r:
            return i, state
    return n - 1, state


def lib_sample(logits, temperature, top_k, top_p, state):
    st, tok = C.c_uint64(state), C.c_uint32()
    check(lib.forge_sample(logits.ctypes.data_as(C.c_void_p), logits.size, temperature, top_k, top_p, C.byref(st), C.byref(tok)))
    return tok.value, st.value


@pytest.mark.parametrize("temperature,top_k,top_p", [(0.0, 0, 0.9), (0.7, 0, 0.9), (1.0, 40, 1.0), (1.3, 5, 0.5), (0.8, 0, 0.0), (0.5, 1, 0.9)])
def test_sample_matches_the_restatement(temperature, top_k, top_p):
    rng = np.random.default_rng(int(temperature * 10) + top_k)
    state = 0xDEADBEEF12345678
    for trial in range(12):
        logits = (rng.standard_normal(300) * 3).astype(np.float32)
        a, b = logits.copy(), logits.copy()
        want, s_ref = ref_sample(a, temperature, top_k, top_p, state)
        got, s_lib = lib_sample(b, temperature, top_k, top_p, state)
        assert got == want and s_lib == s_ref
        assert np.array_equal(a, b)  # the probabilities left behind are the same bits
        state = s_ref if temperature > 0 else state + trial + 1


def test_repeat_penalty_and_argmax_ties():
    logits = np.array([1.0, -2.0, 3.0, 3.0, 0.0], np.float32)
    got, _ = lib_sample(logits.copy(), 0.0, 0, 0.9, 1)
    assert got == 3                                         # the last of equal maxima
    recent = np.array([2, 2, 1, 4, 9], np.uint32)           # twice the same id: penalised twice; 9 is out of range
    a, b = logits.copy(), logits.copy()
    ref_repeat_penalty(a, recent, 1.1)
    check(lib.forge_apply_repeat_penalty(b.ctypes.data_as(C.c_void_p), b.size, recent.ctypes.data_as(C.c_void_p), recent.size, 1.1))
    assert np.array_equal(a, b) and b[2] < 3.0 / 1.1 and b[1] < -2.0
    check(lib.forge_apply_repeat_penalty(b.ctypes.data_as(C.c_void_p), b.size, recent.ctypes.data_as(C.c_void_p), recent.size, 1.0))
    assert np.array_equal(a, b)                             # a penalty of 1 changes nothing


@pytest.mark.gpu
@pytest.mark.parametrize("temperature,top_k", [(0.0, 0), (0.8, 40)])
def test_generate_loop(temperature, top_k):
    from forge_llm_b200 import configs, runtime, synth
    c = configs.tiny(8, hd=64, nq=4, nkv=2, layers=2)
    gm = runtime.Model(c, synth.make_weights_bin(c))
    prompt = synth.prompt_tokens(c, 20).astype(np.uint32)
    sp = ForgeSampling(temperature, top_k, 0.9, 1.1, 0xDEADBEEF12345678)
    # the loop restated on top of forward(): prefill, sample, then [stop at EOS | emit, forward, penalty, sample]
    kv = gm.new_cache(max_seq=80)
    state = sp.seed
    logits = gm.forward_prefill(prompt, kv)
    nxt, state = ref_sample(logits, temperature, top_k, 0.9, state)
    want, recent = [], list(prompt)
    for _ in range(24):
        want.append(nxt)
        recent.append(nxt)
        logits = gm.forward(nxt, kv)
        ref_repeat_penalty(logits, recent, 1.1)
        nxt, state = ref_sample(logits, temperature, top_k, 0.9, state)
    eos = np.array([want[17]], np.uint32)                   # pretend one of the tokens ends the text
    stop = want.index(want[17])
    kv.reset()
    out = np.zeros(24, np.uint32)
    n = C.c_int32()
    check(lib.forge_generate(gm._h, kv._h, prompt.ctypes.data_as(C.c_void_p), prompt.size, 24, C.byref(sp), eos.ctypes.data_as(C.c_void_p), 1,
                             out.ctypes.data_as(C.c_void_p), C.byref(n)))
    assert n.value == stop and list(out[:stop]) == want[:stop]
    kv.close()
    gm.close()

"""Writes tests/golden/tiny_models.npz: outputs of the CPU restatement (oracle/) on seeded tiny models.

    python tests/golden/make_golden.py

The fixtures pin the oracle against drift (CPU test) and give the CUDA path a committed target that does not depend on
building the oracle on the GPU box (GPU test).  Inputs are rebuilt from seeds by forge_llm_b200.synth.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

CASES = {  # name -> arguments of configs.tiny
    "q8_hd64_gqa": dict(quant=8, hd=64, nq=4, nkv=2, layers=2),
    "q4_hd64_gqa": dict(quant=4, hd=64, nq=4, nkv=2, layers=2),
    "q4_hd128_mha_bias": dict(quant=4, hd=128, nq=2, nkv=2, bias=1, layers=3),
    "q8_hd96_gqa": dict(quant=8, hd=96, nq=4, nkv=1, layers=2, hidden=384),
    # K-quants: uniform Q6_K, and the Q4_K_M mix (Q4_K for q/k/o/gate/up, Q6_K for v/down/lm_head); "mix" names the
    # categories configs.with_proj_quant overrides
    "q6k_hd64_gqa": dict(quant=14, hd=64, nq=4, nkv=2, layers=2, ffn=512),
    "q4km_hd64_gqa_bias": dict(quant=12, hd=64, nq=4, nkv=2, layers=2, ffn=512, bias=1, mix=dict(v=14, down=14, lm_head=14)),
}
N_PROMPT, N_NEW = 37, 12


def case_config(name):
    from forge_llm_b200 import configs
    kw = dict(CASES[name])
    mix = kw.pop("mix", None)
    c = configs.tiny(**kw)
    return configs.with_proj_quant(c, **mix) if mix else c


def main():
    from forge_llm_b200 import synth
    from oracle import oracle
    out = {}
    for name in CASES:
        c = case_config(name)
        blob = synth.make_weights_bin(c)
        toks = synth.prompt_tokens(c, N_PROMPT)
        om = oracle.OracleModel(c, blob, kv_mode=oracle.KV_F16)
        logits, trace = om.forward_prefill(toks, trace=True)
        om.reset()
        ids, last = om.generate_greedy(toks, N_NEW)
        out[name + "/prefill_logits"] = logits
        out[name + "/last_hidden"] = trace[-1, -1].copy()
        out[name + "/greedy_ids"] = ids
        out[name + "/final_logits"] = last
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "tiny_models.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()

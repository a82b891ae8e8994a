"""B200 (sm_100a) backend for ForgeLLM's quantized transformer forward path.

``libforge_b200.so`` (hand-written CUDA kernels behind a C ABI, see include/forge_b200.h) is the
product; this package is the thin host-side mirror of the reference's generated ``model::``
surface used by the tests and the benchmark.  Importing ``forge_llm_b200.runtime`` requires the
built library; ``configs`` and ``synth`` are pure numpy.
"""

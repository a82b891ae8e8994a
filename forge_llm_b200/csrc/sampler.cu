// Token selection and the generation loop of the reference's generated main.rs (host code; the logits come back
// from forge_forward like the Vec<f32> of model::forward): argmax / apply_repeat_penalty / sample
// (crates/forgellm-codegen-cpu/src/project.rs:501-551, xorshift RNG :545-548) and the prompt -> tokens loop with its
// EOS stop (:714-751).  The arithmetic keeps the reference's order - sequential f32 sums over the vocabulary, libm
// expf, divisions - so the same seed gives the same tokens.  One latitude is inherited: the reference sorts with
// sort_unstable_by, so the order of exactly equal probabilities is unspecified there too.
#include <algorithm>
#include <cmath>
#include <numeric>
#include <vector>

#include "common.cuh"

namespace {

using namespace forge;

uint32_t argmax_last_host(const float* v, int n) {  // max_by(partial_cmp) keeps the LAST of equal maxima (:501-503)
    int best = 0;
    for (int i = 1; i < n; ++i) if (v[i] >= v[best]) best = i;
    return uint32_t(best);
}

}  // namespace

extern "C" {

int32_t forge_apply_repeat_penalty(float* logits, int32_t n, const uint32_t* recent, size_t n_recent, float penalty) {
    if (!logits || n <= 0 || (!recent && n_recent)) { set_error("bad argument to forge_apply_repeat_penalty"); return FORGE_ERR_INVALID_ARG; }
    if (penalty <= 1.0f) return FORGE_OK;
    for (size_t i = 0; i < n_recent; ++i) {  // once per occurrence, as the reference does (:505-513)
        const uint32_t idx = recent[i];
        if (idx < uint32_t(n)) { if (logits[idx] > 0.0f) logits[idx] /= penalty; else logits[idx] *= penalty; }
    }
    return FORGE_OK;
}

int32_t forge_sample(float* logits, int32_t n, float temperature, int32_t top_k, float top_p, uint64_t* rng_state, uint32_t* token) {
    if (!logits || n <= 0 || !rng_state || !token || top_k < 0) { set_error("bad argument to forge_sample"); return FORGE_ERR_INVALID_ARG; }
    if (temperature <= 0.0f) { *token = argmax_last_host(logits, n); return FORGE_OK; }
    for (int i = 0; i < n; ++i) logits[i] /= temperature;
    float max_val = -INFINITY;
    for (int i = 0; i < n; ++i) max_val = std::max(max_val, logits[i]);
    float sum = 0.0f;
    for (int i = 0; i < n; ++i) { logits[i] = std::exp(logits[i] - max_val); sum += logits[i]; }
    for (int i = 0; i < n; ++i) logits[i] /= sum;
    std::vector<int> order(n);
    std::iota(order.begin(), order.end(), 0);
    std::sort(order.begin(), order.end(), [&](int a, int b) { return logits[a] > logits[b]; });  // descending probability
    if (top_k > 0 && top_k < n)
        for (int i = top_k; i < n; ++i) logits[order[i]] = 0.0f;
    if (top_p > 0.0f && top_p < 1.0f) {
        float cumsum = 0.0f;
        for (int i = 0; i < n; ++i) {  // every entry at which the running sum has passed top_p is dropped (:531-539)
            cumsum += logits[order[i]];
            if (cumsum > top_p) logits[order[i]] = 0.0f;
        }
    }
    sum = 0.0f;
    for (int i = 0; i < n; ++i) sum += logits[i];
    if (sum > 0.0f) for (int i = 0; i < n; ++i) logits[i] /= sum;
    uint64_t s = *rng_state;
    s ^= s << 13; s ^= s >> 7; s ^= s << 17;
    *rng_state = s;
    const float r = float(s) / 18446744073709551616.0f;  // u64::MAX as f32 rounds to 2^64
    float cumsum = 0.0f;
    for (int i = 0; i < n; ++i) {
        cumsum += logits[i];
        if (cumsum >= r) { *token = uint32_t(i); return FORGE_OK; }
    }
    *token = uint32_t(n - 1);
    return FORGE_OK;
}

int32_t forge_generate(ForgeModel* model, ForgeKV* kv, const uint32_t* prompt, size_t n_prompt, int32_t max_tokens,
                       const ForgeSampling* sp, const uint32_t* eos, size_t n_eos, uint32_t* out_tokens, int32_t* n_out) {
    if (!model || !kv || !prompt || n_prompt == 0 || max_tokens < 0 || !sp || !out_tokens || !n_out || (!eos && n_eos)) { set_error("bad argument to forge_generate"); return FORGE_ERR_INVALID_ARG; }
    *n_out = 0;
    const size_t V = forge_model_vocab_size(model);
    std::vector<float> logits(V);
    uint64_t rng = sp->seed;
    FORGE_TRY(forge_forward_prefill(model, kv, prompt, n_prompt, logits.data()));
    uint32_t next = 0;
    FORGE_TRY(forge_sample(logits.data(), int32_t(V), sp->temperature, sp->top_k, sp->top_p, &rng, &next));
    std::vector<uint32_t> recent(prompt, prompt + n_prompt);
    for (int32_t i = 0; i < max_tokens; ++i) {
        if (std::find(eos, eos + n_eos, next) != eos + n_eos) break;
        out_tokens[(*n_out)++] = next;
        recent.push_back(next);
        FORGE_TRY(forge_forward(model, kv, next, logits.data()));
        FORGE_TRY(forge_apply_repeat_penalty(logits.data(), int32_t(V), recent.data(), recent.size(), sp->repeat_penalty));
        FORGE_TRY(forge_sample(logits.data(), int32_t(V), sp->temperature, sp->top_k, sp->top_p, &rng, &next));
    }
    return FORGE_OK;
}

}  // extern "C"

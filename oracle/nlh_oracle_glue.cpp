// CPU oracle, block glue: LayerNorm, cross-entropy, embedding gather / scatter-add.
// TEST INFRASTRUCTURE ONLY: nothing in the product path may call into this file.
//
// Restates the reference's CPU code (plain loops, same accumulation order):
//   layer_norm / layer_norm_backward        core/src/mag.rs:396-449
//   cross_entropy_loss                      core/src/tensor.rs:167-198
//   cross-entropy gradient (softmax - onehot) * inv_count, zero rows for invalid targets
//                                           core/kernels/cross_entropy.cu:99-160 (the only statement)
//   embedding gather / scatter-add          core/kernels/embedding.cu:20-94
// Parity pins: closed-form numpy float64 checks and finite differences in tests/test_oracle.py
// (the reference holds no golden vectors for these functions).
#include <cmath>
#include <cstdint>
#include <cstring>

#define ORC_API extern "C" __attribute__((visibility("default")))

ORC_API void orc_layer_norm_forward(const float* x, const float* gamma, const float* beta,
                                    float* out, float* mean_cache, float* rstd_cache,
                                    int n, int d, float eps) {
    for (int i = 0; i < n; i++) {
        const float* row = x + (int64_t)i * d;
        float sum = 0.0f;
        for (int j = 0; j < d; j++) sum += row[j];
        const float mean = sum / (float)d;
        float vs = 0.0f;
        for (int j = 0; j < d; j++) vs += (row[j] - mean) * (row[j] - mean);
        const float var = vs / (float)d;
        const float rstd = 1.0f / std::sqrt(var + eps);
        mean_cache[i] = mean;
        rstd_cache[i] = rstd;
        for (int j = 0; j < d; j++) out[(int64_t)i * d + j] = gamma[j] * (row[j] - mean) * rstd + beta[j];
    }
}

// d_gamma / d_beta are accumulated into (caller zeroes), as in the reference's GPU entry.
ORC_API void orc_layer_norm_backward(const float* d_out, const float* x, const float* gamma,
                                     const float* mean_cache, const float* rstd_cache,
                                     float* d_x, float* d_gamma, float* d_beta, int n, int d) {
    const float d_f = (float)d;
    for (int i = 0; i < n; i++) {
        const float mean = mean_cache[i], rstd = rstd_cache[i];
        float sum1 = 0.0f, sum2 = 0.0f;
        for (int j = 0; j < d; j++) {
            const float x_hat = (x[(int64_t)i * d + j] - mean) * rstd;
            const float dy = d_out[(int64_t)i * d + j];
            d_gamma[j] += dy * x_hat;
            d_beta[j] += dy;
            sum1 += dy * gamma[j];
            sum2 += dy * gamma[j] * x_hat;
        }
        for (int j = 0; j < d; j++) {
            const float x_hat = (x[(int64_t)i * d + j] - mean) * rstd;
            d_x[(int64_t)i * d + j] =
                rstd / d_f * (d_f * d_out[(int64_t)i * d + j] * gamma[j] - sum1 - x_hat * sum2);
        }
    }
}

// Returns the SUM of the per-position negative log-likelihoods and the number of valid targets
// (the reference's CPU function divides, its GPU entry returns the sum).
ORC_API float orc_cross_entropy_sum(const float* logits, const int32_t* targets, int seq_len,
                                    int vocab, int* count_out) {
    float total = 0.0f;
    int count = 0;
    for (int t = 0; t < seq_len; t++) {
        const float* row = logits + (int64_t)t * vocab;
        const int target = targets[t];
        if (target < 0 || target >= vocab) continue;
        float max_val = -INFINITY;
        for (int v = 0; v < vocab; v++) max_val = row[v] > max_val ? row[v] : max_val;
        float sum_exp = 0.0f;
        for (int v = 0; v < vocab; v++) sum_exp += std::exp(row[v] - max_val);
        const float log_softmax = (row[target] - max_val) - std::log(sum_exp);
        total -= log_softmax;
        count++;
    }
    if (count_out) *count_out = count;
    return total;
}

ORC_API void orc_cross_entropy_backward(const float* logits, const int32_t* targets, float* d_logits,
                                        int seq_len, int vocab, float inv_count) {
    for (int t = 0; t < seq_len; t++) {
        const float* row = logits + (int64_t)t * vocab;
        float* drow = d_logits + (int64_t)t * vocab;
        const int target = targets[t];
        if (target < 0 || target >= vocab) {
            for (int v = 0; v < vocab; v++) drow[v] = 0.0f;
            continue;
        }
        float max_val = -INFINITY;
        for (int v = 0; v < vocab; v++) max_val = row[v] > max_val ? row[v] : max_val;
        float sum_exp = 0.0f;
        for (int v = 0; v < vocab; v++) sum_exp += std::exp(row[v] - max_val);
        for (int v = 0; v < vocab; v++) {
            const float p = std::exp(row[v] - max_val) / sum_exp;
            drow[v] = (p - (v == target ? 1.0f : 0.0f)) * inv_count;
        }
    }
}

ORC_API void orc_embedding_gather(const float* w_embed, const int32_t* ids, float* out, int seq_len, int d) {
    for (int t = 0; t < seq_len; t++)
        std::memcpy(out + (int64_t)t * d, w_embed + (int64_t)ids[t] * d, sizeof(float) * d);
}

ORC_API void orc_embedding_scatter_add(const float* d_embedded, const int32_t* ids, float* d_embed,
                                       int seq_len, int d) {
    for (int t = 0; t < seq_len; t++)
        for (int j = 0; j < d; j++) d_embed[(int64_t)ids[t] * d + j] += d_embedded[(int64_t)t * d + j];
}

/*
 * CPU restatement of the NERVE compute shaders that lie on the MTP speculative
 * decode path.  TEST INFRASTRUCTURE ONLY: this file is the parity checker and
 * the timed CPU baseline; the product never links, loads or calls it.
 *
 * Parity status: the reference ships no golden logits / token sequences for
 * this path ("parity unpinned" for numerics).  What the reference's own tests
 * pin - the acceptance rule, the greedy sampler record, the seeded sampler
 * hash, the control/page-table byte layouts, the bf16/e4m3 conversions - is
 * checked against this file in tests/test_oracle_pins.py.
 *
 * Every function cites the shader (runtime-rs/shaders/...) it follows.  All
 * activations are bf16 bit patterns (uint16_t), row-major [lane][width];
 * accumulation is f32 with the same rounding points as the shader:
 *   bf16 rounding = (bits + 0x7fff + lsb) >> 16 with no NaN special case.
 * The reduction ORDER inside a dot product mirrors the shaders' shape
 * (64 strided lane partials, then a sum over lanes) but subgroup-tree order is
 * implementation-defined in the reference, so order is not a parity criterion.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

static inline float bf2f(uint16_t v) {
    uint32_t bits = (uint32_t)v << 16;
    float out;
    memcpy(&out, &bits, 4);
    return out;
}

static inline uint16_t f2bf(float value) {
    uint32_t bits;
    memcpy(&bits, &value, 4);
    uint32_t lsb = (bits >> 16) & 1u;
    return (uint16_t)((bits + 0x7fffu + lsb) >> 16);
}

static inline float rbf(float value) { return bf2f(f2bf(value)); }

ORC_API uint16_t orc_f32_to_bf16(float value) { return f2bf(value); }
ORC_API float orc_bf16_to_f32(uint16_t value) { return bf2f(value); }

/* ---- e4m3 (fn variant: no inf, 0x7f/0xff = NaN, max 448) ------------------ */

static float E4M3_TABLE[256];
static int e4m3_ready = 0;

static void e4m3_init(void) {
    if (e4m3_ready) return;
    for (int code = 0; code < 256; code++) {
        int exponent = (code >> 3) & 0xf, mantissa = code & 7;
        float value;
        if (exponent == 0xf && mantissa == 7) value = NAN;
        else if (exponent == 0) value = ldexpf((float)mantissa / 8.0f, -6);
        else value = ldexpf(1.0f + (float)mantissa / 8.0f, exponent - 7);
        E4M3_TABLE[code] = (code & 0x80) ? -value : value;
    }
    e4m3_ready = 1;
}

ORC_API float orc_e4m3_to_f32(uint8_t code) {
    e4m3_init();
    return E4M3_TABLE[code];
}

/* f32 -> e4m3fn, round-to-nearest-even, saturating at 448 (the shaders only
 * convert values already scaled into [-448, 448]). */
ORC_API uint8_t orc_f32_to_e4m3(float value) {
    uint8_t sign = signbit(value) ? 0x80 : 0;
    float mag = fabsf(value);
    if (isnan(mag)) return sign | 0x7f;
    if (mag >= 448.0f) return sign | 0x7e;
    if (mag == 0.0f) return sign;
    int exponent;
    (void)frexpf(mag, &exponent); /* mag = m * 2^exponent, m in [0.5,1) */
    exponent -= 1;                /* mag = (1.x) * 2^exponent */
    if (exponent < -6) exponent = -6;
    float quantum = ldexpf(1.0f, exponent - 3);
    float steps = rintf(mag / quantum); /* default rounding mode: ties-to-even */
    float q = steps * quantum;
    if (q >= 448.0f) return sign | 0x7e;
    if (q == 0.0f) return sign;
    (void)frexpf(q, &exponent);
    exponent -= 1;
    if (exponent < -6) {
        int mantissa = (int)(q / ldexpf(1.0f, -9));
        return sign | (uint8_t)mantissa;
    }
    int mantissa = (int)((q / ldexpf(1.0f, exponent) - 1.0f) * 8.0f);
    return sign | (uint8_t)(((exponent + 7) << 3) | mantissa);
}

/* ---- rms_norm_bf16.comp.template:49-72 ----------------------------------- */
ORC_API void orc_rms_norm(const uint16_t *x, const uint16_t *w, uint16_t *y, int lanes, int width,
                          float eps, float weight_offset) {
#pragma omp parallel for if (lanes > 1)
    for (int m = 0; m < lanes; m++) {
        const uint16_t *row = x + (size_t)m * width;
        float partial[64];
        for (int lane = 0; lane < 64; lane++) partial[lane] = 0.0f;
        for (int i = 0; i < width; i++) {
            float value = bf2f(row[i]);
            partial[i & 63] = fmaf(value, value, partial[i & 63]);
        }
        float sum = 0.0f;
        for (int lane = 0; lane < 64; lane++) sum += partial[lane];
        float inv_rms = 1.0f / sqrtf(sum / (float)width + eps);
        for (int i = 0; i < width; i++) {
            float value = bf2f(row[i]) * inv_rms * (bf2f(w[i]) + weight_offset);
            y[(size_t)m * width + i] = f2bf(value);
        }
    }
}

/* ---- dot products --------------------------------------------------------- */

static inline float dot_bf16(const uint16_t *x, const uint16_t *w, int k) {
    /* linear_bf16.comp.template:49-64: lane l handles word l, l+64, ...;
     * each word is two fma's (low half then high half). */
    float partial[64];
    for (int lane = 0; lane < 64; lane++) partial[lane] = 0.0f;
    int words = k / 2;
    for (int word = 0; word < words; word++) {
        int lane = word & 63;
        partial[lane] = fmaf(bf2f(x[2 * word]), bf2f(w[2 * word]), partial[lane]);
        partial[lane] = fmaf(bf2f(x[2 * word + 1]), bf2f(w[2 * word + 1]), partial[lane]);
    }
    if (k & 1) partial[words & 63] = fmaf(bf2f(x[k - 1]), bf2f(w[k - 1]), partial[words & 63]);
    float sum = 0.0f;
    for (int lane = 0; lane < 64; lane++) sum += partial[lane];
    return sum;
}

/* linear_bf16.comp.template:38-95 (one bf16 rounding). */
ORC_API void orc_linear_bf16(const uint16_t *x, const uint16_t *w, uint16_t *y, int lanes, int n, int k) {
#pragma omp parallel for schedule(static)
    for (int row = 0; row < n; row++) {
        const uint16_t *wr = w + (size_t)row * k;
        for (int m = 0; m < lanes; m++)
            y[(size_t)m * n + row] = f2bf(dot_bf16(x + (size_t)m * k, wr, k));
    }
}

/* linear_residual_bf16.comp.template:47-53: round the product to bf16, add the
 * residual in f32, round again. */
ORC_API void orc_linear_residual_bf16(const uint16_t *x, const uint16_t *w, const uint16_t *residual,
                                      uint16_t *y, int lanes, int n, int k) {
#pragma omp parallel for schedule(static)
    for (int row = 0; row < n; row++) {
        const uint16_t *wr = w + (size_t)row * k;
        for (int m = 0; m < lanes; m++) {
            float product = rbf(dot_bf16(x + (size_t)m * k, wr, k));
            y[(size_t)m * n + row] = f2bf(product + bf2f(residual[(size_t)m * n + row]));
        }
    }
}

static inline float rounded_silu(float value) { return rbf(value / (1.0f + expf(-value))); }

/* parallel_linear_silu_multiply_bf16.comp.template:58-72: gate and up are each
 * rounded to bf16, SiLU(gate) is rounded, the product is rounded. */
ORC_API void orc_linear_silu_multiply_bf16(const uint16_t *x, const uint16_t *wg, const uint16_t *wu,
                                           uint16_t *y, int lanes, int n, int k) {
#pragma omp parallel for schedule(static)
    for (int row = 0; row < n; row++) {
        for (int m = 0; m < lanes; m++) {
            float gate = rbf(dot_bf16(x + (size_t)m * k, wg + (size_t)row * k, k));
            float up = rbf(dot_bf16(x + (size_t)m * k, wu + (size_t)row * k, k));
            y[(size_t)m * n + row] = f2bf(rounded_silu(gate) * up);
        }
    }
}

/* linear_int4_ct.comp.template:80-150.  qweight[row][k/8] (nibble j of a word
 * is column 8*word+j, low nibble first, value-8), scales bf16 [row][k/group].
 * Lane l handles packed words l, l+64, ...; per word:
 *   sum = fma(dot(x[0..3], w_lo) + dot(x[4..7], w_hi), scale, sum). */
ORC_API void orc_linear_int4_ct(const uint16_t *x, const uint32_t *qweight, const uint16_t *scales,
                                uint16_t *y, int lanes, int n, int k, int group) {
    int packed_columns = k / 8, scale_columns = k / group;
    float *xf = (float *)malloc(sizeof(float) * (size_t)lanes * k);
    for (size_t i = 0; i < (size_t)lanes * k; i++) xf[i] = bf2f(x[i]);
#pragma omp parallel for schedule(static)
    for (int row = 0; row < n; row++) {
        const uint32_t *qr = qweight + (size_t)row * packed_columns;
        const uint16_t *sr = scales + (size_t)row * scale_columns;
        for (int m = 0; m < lanes; m++) {
            const float *xm = xf + (size_t)m * k;
            float partial[64];
            for (int lane = 0; lane < 64; lane++) partial[lane] = 0.0f;
            for (int pc = 0; pc < packed_columns; pc++) {
                uint32_t packed = qr[pc];
                const float *xs = xm + pc * 8;
                float lo = xs[0] * (float)((int)(packed & 15u) - 8);
                lo += xs[1] * (float)((int)((packed >> 4) & 15u) - 8);
                lo += xs[2] * (float)((int)((packed >> 8) & 15u) - 8);
                lo += xs[3] * (float)((int)((packed >> 12) & 15u) - 8);
                float hi = xs[4] * (float)((int)((packed >> 16) & 15u) - 8);
                hi += xs[5] * (float)((int)((packed >> 20) & 15u) - 8);
                hi += xs[6] * (float)((int)((packed >> 24) & 15u) - 8);
                hi += xs[7] * (float)((int)((packed >> 28) & 15u) - 8);
                float scale = bf2f(sr[(pc * 8) / group]);
                partial[pc & 63] = fmaf(lo + hi, scale, partial[pc & 63]);
            }
            float sum = 0.0f;
            for (int lane = 0; lane < 64; lane++) sum += partial[lane];
            y[(size_t)m * n + row] = f2bf(sum);
        }
    }
    free(xf);
}

/* add_bf16.comp.template:17-24 */
ORC_API void orc_add_bf16(const uint16_t *a, const uint16_t *b, uint16_t *y, size_t count) {
    for (size_t i = 0; i < count; i++) y[i] = f2bf(bf2f(a[i]) + bf2f(b[i]));
}

/* silu_multiply_bf16.comp.template:30-52 */
ORC_API void orc_silu_multiply(const uint16_t *gate, const uint16_t *up, uint16_t *y, size_t count) {
    for (size_t i = 0; i < count; i++) y[i] = f2bf(rounded_silu(bf2f(gate[i])) * bf2f(up[i]));
}

/* rotary_bf16.comp.template:50-109, half-split / interleaved, no YaRN
 * (attention factor 1).  position = low 32 bits of the stream tick. */
static inline float rope_rotate(const uint16_t *head, int dim, int rotary, int interleaved, float theta,
                                uint32_t position) {
    if (dim >= rotary) return bf2f(head[dim]);
    int half = rotary / 2;
    int frequency_index = interleaved ? dim / 2 : dim % half;
    float inv_freq = powf(theta, -2.0f * (float)frequency_index / (float)rotary);
    float angle = (float)position * inv_freq;
    float cosine = rbf(cosf(angle) * 1.0f);
    float sine = rbf(sinf(angle) * 1.0f);
    float other;
    if (interleaved) other = (dim & 1) == 0 ? -bf2f(head[dim + 1]) : bf2f(head[dim - 1]);
    else other = dim < half ? -bf2f(head[dim + half]) : bf2f(head[dim - half]);
    float direct = rbf(bf2f(head[dim]) * cosine);
    float rotated = rbf(other * sine);
    return rbf(direct + rotated);
}

ORC_API void orc_rotary(const uint16_t *x, uint16_t *y, const uint32_t *positions, int lanes, int heads,
                        int head_width, int rotary, int interleaved, float theta) {
    for (int m = 0; m < lanes; m++)
        for (int h = 0; h < heads; h++) {
            const uint16_t *head = x + ((size_t)m * heads + h) * head_width;
            uint16_t *out = y + ((size_t)m * heads + h) * head_width;
            for (int d = 0; d < head_width; d++)
                out[d] = f2bf(rope_rotate(head, d, rotary, interleaved, theta, positions[m]));
        }
}

/* parallel_head_norm_rope_2way_bf16.comp.template:166-209: per-head RMSNorm
 * (rounded to bf16) followed by RoPE on the rounded values. */
ORC_API void orc_head_norm_rope(const uint16_t *x, const uint16_t *norm_weight, uint16_t *y,
                                const uint32_t *positions, int lanes, int heads, int head_width, int rotary,
                                int interleaved, float theta, float eps, float weight_offset) {
    uint16_t *normalized = (uint16_t *)malloc(sizeof(uint16_t) * head_width);
    for (int m = 0; m < lanes; m++)
        for (int h = 0; h < heads; h++) {
            const uint16_t *head = x + ((size_t)m * heads + h) * head_width;
            float partial[64];
            for (int lane = 0; lane < 64; lane++) partial[lane] = 0.0f;
            for (int d = 0; d < head_width; d++) {
                float value = bf2f(head[d]);
                partial[d & 63] = fmaf(value, value, partial[d & 63]);
            }
            float sum = 0.0f;
            for (int lane = 0; lane < 64; lane++) sum += partial[lane];
            float inv_rms = 1.0f / sqrtf(sum / (float)head_width + eps);
            for (int d = 0; d < head_width; d++)
                normalized[d] = f2bf(bf2f(head[d]) * inv_rms * (bf2f(norm_weight[d]) + weight_offset));
            uint16_t *out = y + ((size_t)m * heads + h) * head_width;
            for (int d = 0; d < head_width; d++)
                out[d] = f2bf(rope_rotate(normalized, d, rotary, interleaved, theta, positions[m]));
        }
    free(normalized);
}

/* append_gqa_attention_bf16.comp.template:171-339 for ONE lane (tick):
 * writes K,V of this tick at ring slot tick % capacity, then attends over
 * min(tick+1, capacity) tokens in chronological order with online softmax in
 * f32 (tiles of `tile_tokens`, as the shader) and one bf16 rounding at the
 * end.  kv_state is the logical (un-paged) ring [capacity][2*kv_heads*hd]. */
ORC_API void orc_append_attention(const uint16_t *q, const uint16_t *k, const uint16_t *v, uint16_t *kv_state,
                                  uint16_t *out, uint32_t tick, uint32_t capacity, int q_heads, int kv_heads,
                                  int head_width, float scale, int tile_tokens) {
    int kv_elements = kv_heads * head_width;
    size_t slot_elements = (size_t)kv_elements * 2;
    if (capacity == 0) {
        memset(out, 0, sizeof(uint16_t) * q_heads * head_width);
        return;
    }
    uint32_t slot_now = tick % capacity;
    memcpy(kv_state + slot_now * slot_elements, k, sizeof(uint16_t) * kv_elements);
    memcpy(kv_state + slot_now * slot_elements + kv_elements, v, sizeof(uint16_t) * kv_elements);
    uint32_t tokens = tick + 1u < capacity ? tick + 1u : capacity;
    uint32_t start = (tick + capacity + 1u - tokens) % capacity;
    int groups = q_heads / kv_heads;
#pragma omp parallel for if (tokens > 256)
    for (int qh = 0; qh < q_heads; qh++) {
        int kvh = qh / groups;
        float *acc = (float *)calloc(head_width, sizeof(float));
        float *alpha = (float *)malloc(sizeof(float) * tile_tokens);
        float *beta = (float *)malloc(sizeof(float) * tile_tokens);
        float *weight = (float *)malloc(sizeof(float) * tile_tokens);
        float maximum = -3.4028234663852886e38f, denominator = 0.0f;
        const uint16_t *qv = q + (size_t)qh * head_width;
        for (uint32_t tile_start = 0; tile_start < tokens; tile_start += tile_tokens) {
            uint32_t tile_count = tokens - tile_start < (uint32_t)tile_tokens ? tokens - tile_start : (uint32_t)tile_tokens;
            for (uint32_t i = 0; i < tile_count; i++) {
                uint32_t slot = start + tile_start + i;
                if (slot >= capacity) slot -= capacity;
                const uint16_t *kr = kv_state + slot * slot_elements + (size_t)kvh * head_width;
                float dot = 0.0f;
                for (int d = 0; d < head_width; d++) dot += bf2f(qv[d]) * bf2f(kr[d]);
                float score = dot * scale;
                float next_maximum = fmaxf(maximum, score);
                alpha[i] = expf(maximum - next_maximum);
                beta[i] = expf(score - next_maximum);
                denominator = denominator * alpha[i] + beta[i];
                maximum = next_maximum;
            }
            float carry = 1.0f;
            for (uint32_t r = tile_count; r > 0; r--) {
                weight[r - 1] = beta[r - 1] * carry;
                carry *= alpha[r - 1];
            }
            for (int d = 0; d < head_width; d++) {
                float tile_sum = 0.0f;
                for (uint32_t i = 0; i < tile_count; i++) {
                    uint32_t slot = start + tile_start + i;
                    if (slot >= capacity) slot -= capacity;
                    const uint16_t *vr = kv_state + slot * slot_elements + kv_elements + (size_t)kvh * head_width;
                    tile_sum += weight[i] * bf2f(vr[d]);
                }
                acc[d] = acc[d] * carry + tile_sum;
            }
        }
        for (int d = 0; d < head_width; d++)
            out[(size_t)qh * head_width + d] = f2bf(denominator == 0.0f ? 0.0f : acc[d] / denominator);
        free(acc);
        free(alpha);
        free(beta);
        free(weight);
    }
}

/* embedding_lookup_bf16.comp.template:31-46 */
ORC_API void orc_embedding(const uint16_t *table, const uint32_t *tokens, uint16_t *y, int lanes, int width,
                           int vocab, float scale) {
    for (int m = 0; m < lanes; m++) {
        if (tokens[m] >= (uint32_t)vocab) continue;
        for (int i = 0; i < width; i++)
            y[(size_t)m * width + i] = f2bf(bf2f(table[(size_t)tokens[m] * width + i]) * scale);
    }
}

/* tied_output_projection_bf16.comp.template:33-91: f32 logits = dot * scale. */
ORC_API void orc_output_projection(const uint16_t *x, const uint16_t *w, float *logits, int lanes, int vocab,
                                   int k, float scale) {
#pragma omp parallel for schedule(static)
    for (int row = 0; row < vocab; row++)
        for (int m = 0; m < lanes; m++)
            logits[(size_t)m * vocab + row] = dot_bf16(x + (size_t)m * k, w + (size_t)row * k, k) * scale;
}

/* greedy_sampler_f32.comp.template:31-34,52-109: arg-max, ties -> lowest id.
 * record = {token, logit bits, 0, 0}. */
ORC_API uint32_t orc_greedy(const float *logits, int vocab, uint32_t *record) {
    uint32_t best = 0;
    float best_logit = vocab > 0 ? logits[0] : -3.4028234663852886e38f;
    for (int token = 1; token < vocab; token++) {
        float candidate = logits[token];
        if (candidate > best_logit) {
            best_logit = candidate;
            best = (uint32_t)token;
        }
    }
    if (record) {
        memcpy(&record[1], &best_logit, 4);
        record[0] = best;
        record[2] = 0;
        record[3] = 0;
    }
    return best;
}

/* temperature_top_k_candidates_f32.comp.template:48-127 + temperature_top_k_top_p_sampler_f32.comp.template:
 * 56-72,100-216: exact top-k of the logits (NaNs skipped; order: larger logit first, ties -> lower id), then
 *   max_scaled = top[0]/T;  min_logit = min_p > 0 ? top[0] + T*log(min_p) : lowest float
 *   total   = sum of exp(l/T - max_scaled) over the list until an entry falls below min_logit
 *   nucleus = the shortest prefix whose weight reaches top_p * total
 *   u       = (hash_u32(seed ^ tick_lo ^ tick_hi*0x9e3779b9) >> 8) * 2^-24;  target = u * nucleus weight
 *   pick the first index whose cumulative weight exceeds target (else the last of the nucleus)
 * record = {token, logit bits, 1, 0}.  All sums in f32 and in list order, as the single shader thread does. */
ORC_API uint32_t orc_hash_u32(uint32_t value) {
    value ^= value >> 16;
    value *= 0x7feb352du;
    value ^= value >> 15;
    value *= 0x846ca68bu;
    value ^= value >> 16;
    return value;
}

ORC_API uint32_t orc_sample_top_k_top_p(const float *logits, int vocab, int top_k, float temperature, float top_p,
                                        float min_p, uint32_t seed, uint32_t tick_lo, uint32_t tick_hi, uint32_t *record) {
    const float lowest = -3.4028234663852886e38f;
    if (top_k < 1) top_k = 1;
    float *top_logit = (float *)malloc(sizeof(float) * (size_t)top_k);
    uint32_t *top_token = (uint32_t *)malloc(sizeof(uint32_t) * (size_t)top_k);
    float previous_logit = 0.0f;
    uint32_t previous_token = 0;
    for (int rank = 0; rank < top_k; rank++) {
        float best = lowest;
        uint32_t best_token = 0xffffffffu;
        for (int token = 0; token < vocab; token++) {
            float candidate = logits[token];
            if (isnan(candidate)) continue;
            if (rank != 0 && !(candidate < previous_logit || (candidate == previous_logit && (uint32_t)token > previous_token)))
                continue;
            if (candidate > best || (candidate == best && (uint32_t)token < best_token)) {
                best = candidate;
                best_token = (uint32_t)token;
            }
        }
        top_logit[rank] = best;
        top_token[rank] = best_token;
        previous_logit = best;
        previous_token = best_token;
    }
    const float max_scaled = top_logit[0] / temperature;
    const float min_logit = min_p > 0.0f ? top_logit[0] + temperature * logf(min_p) : lowest;
    float total = 0.0f;
    for (int i = 0; i < top_k; i++) {
        if (top_logit[i] < min_logit) break;
        total += expf(top_logit[i] / temperature - max_scaled);
    }
    const float threshold = top_p * total;
    float nucleus = 0.0f;
    int count = 0;
    for (int i = 0; i < top_k; i++) {
        if (top_logit[i] < min_logit) break;
        nucleus += expf(top_logit[i] / temperature - max_scaled);
        count = i + 1;
        if (nucleus >= threshold) break;
    }
    const uint32_t bits = orc_hash_u32(seed ^ tick_lo ^ (tick_hi * 0x9e3779b9u));
    const float target = (float)(bits >> 8) * (1.0f / 16777216.0f) * nucleus;
    float cumulative = 0.0f;
    int selected = count - 1;
    for (int i = 0; i < count; i++) {
        cumulative += expf(top_logit[i] / temperature - max_scaled);
        if (target < cumulative) {
            selected = i;
            break;
        }
    }
    if (selected < 0) selected = 0;
    const uint32_t token = top_token[selected];
    if (record) {
        record[0] = token;
        memcpy(&record[1], &top_logit[selected], 4);
        record[2] = 1;
        record[3] = 0;
    }
    free(top_logit);
    free(top_token);
    return token;
}

/* Top-2 gap of a logits row (used by the parity rule "divergence allowed only
 * where the oracle's top-2 gap is below 1e-3"). */
ORC_API float orc_top2_gap(const float *logits, int vocab) {
    float first = -INFINITY, second = -INFINITY;
    for (int token = 0; token < vocab; token++) {
        float value = logits[token];
        if (value > first) {
            second = first;
            first = value;
        } else if (value > second) {
            second = value;
        }
    }
    return first - second;
}

/* ---- FP8 W8A8 ------------------------------------------------------------- */

/* quantize_fp8_e4m3.comp.template:41-60: per 128-column block
 * scale = absmax/448 (1 if absmax == 0), q = e4m3(x / scale). */
ORC_API void orc_quantize_fp8(const uint16_t *x, uint8_t *q, float *scales, int lanes, int k, int block) {
    e4m3_init();
    int blocks = k / block;
    for (int m = 0; m < lanes; m++)
        for (int b = 0; b < blocks; b++) {
            const uint16_t *xs = x + (size_t)m * k + (size_t)b * block;
            float absmax = 0.0f;
            for (int i = 0; i < block; i++) absmax = fmaxf(absmax, fabsf(bf2f(xs[i])));
            float scale = absmax > 0.0f ? absmax / 448.0f : 1.0f;
            scales[(size_t)m * blocks + b] = scale;
            for (int i = 0; i < block; i++)
                q[(size_t)m * k + (size_t)b * block + i] = orc_f32_to_e4m3(bf2f(xs[i]) / scale);
        }
}

static inline float dot_fp8(const uint8_t *xq, const float *xscale, const uint8_t *wrow, const uint16_t *wscale_row,
                            int k, int block) {
    /* linear_prequant_fp8_e4m3.comp.template:82-108: per 4 elements an exact
     * f32 dot, then fma(dot4, act_scale*weight_scale, sum); lane = word % 64. */
    float partial[64];
    for (int lane = 0; lane < 64; lane++) partial[lane] = 0.0f;
    int words = k / 4;
    for (int word = 0; word < words; word++) {
        int b = (word * 4) / block;
        float d = 0.0f;
        for (int j = 0; j < 4; j++) d += E4M3_TABLE[xq[word * 4 + j]] * E4M3_TABLE[wrow[word * 4 + j]];
        partial[word & 63] = fmaf(d, xscale[b] * bf2f(wscale_row[b]), partial[word & 63]);
    }
    float sum = 0.0f;
    for (int lane = 0; lane < 64; lane++) sum += partial[lane];
    return sum;
}

/* Prequantised FP8 linear; residual (optional) is added in f32 BEFORE the one
 * bf16 rounding (linear_residual_fp8_e4m3 finalize_output,
 * nerve/model_package_shader_templates.py:746-783). weight_scale_inv bf16
 * [ceil(n/block_rows)][k/block]. */
ORC_API void orc_linear_fp8(const uint8_t *xq, const float *xscales, const uint8_t *w, const uint16_t *wscale,
                            const uint16_t *residual, uint16_t *y, int lanes, int n, int k, int block_rows,
                            int block) {
    e4m3_init();
    int blocks = k / block;
#pragma omp parallel for schedule(static)
    for (int row = 0; row < n; row++) {
        const uint16_t *ws = wscale + (size_t)(row / block_rows) * blocks;
        for (int m = 0; m < lanes; m++) {
            float sum = dot_fp8(xq + (size_t)m * k, xscales + (size_t)m * blocks, w + (size_t)row * k, ws, k, block);
            if (residual) sum = bf2f(residual[(size_t)m * n + row]) + sum;
            y[(size_t)m * n + row] = f2bf(sum);
        }
    }
}

/* parallel_linear_silu_multiply_prequant_fp8: gate/up rounded to bf16, SiLU
 * rounded, product rounded (same chain as the bf16 form). */
ORC_API void orc_linear_silu_multiply_fp8(const uint8_t *xq, const float *xscales, const uint8_t *wg,
                                          const uint16_t *wg_scale, const uint8_t *wu, const uint16_t *wu_scale,
                                          uint16_t *y, int lanes, int n, int k, int block_rows, int block) {
    e4m3_init();
    int blocks = k / block;
#pragma omp parallel for schedule(static)
    for (int row = 0; row < n; row++) {
        for (int m = 0; m < lanes; m++) {
            float gate = rbf(dot_fp8(xq + (size_t)m * k, xscales + (size_t)m * blocks, wg + (size_t)row * k,
                                     wg_scale + (size_t)(row / block_rows) * blocks, k, block));
            float up = rbf(dot_fp8(xq + (size_t)m * k, xscales + (size_t)m * blocks, wu + (size_t)row * k,
                                   wu_scale + (size_t)(row / block_rows) * blocks, k, block));
            y[(size_t)m * n + row] = f2bf(rounded_silu(gate) * up);
        }
    }
}

/* ---- MoE ------------------------------------------------------------------ */

/* moe_topk_bf16.comp.template:42-84: k rounds of arg-max (first max wins),
 * softmax over the selected logits in score order, routes then sorted by
 * expert id; word = bf16(weight) << 16 | expert. */
ORC_API void orc_moe_topk(const uint16_t *router_logits, uint32_t *routes, int lanes, int experts, int top_k) {
    for (int m = 0; m < lanes; m++) {
        const uint16_t *logits = router_logits + (size_t)m * experts;
        uint32_t *out = routes + (size_t)m * top_k;
        int selected[64];
        for (int route = 0; route < top_k; route++) {
            float best_score = -INFINITY;
            int best = 0;
            for (int e = 0; e < experts; e++) {
                int taken = 0;
                for (int i = 0; i < route; i++) taken |= selected[i] == e;
                float score = bf2f(logits[e]);
                if (!taken && score > best_score) {
                    best_score = score;
                    best = e;
                }
            }
            selected[route] = best;
        }
        float maximum = bf2f(logits[selected[0]]);
        float denominator = 0.0f;
        for (int route = 0; route < top_k; route++) denominator += expf(bf2f(logits[selected[route]]) - maximum);
        for (int route = 1; route < top_k; route++) {
            int e = selected[route], ins = route;
            while (ins > 0 && selected[ins - 1] > e) {
                selected[ins] = selected[ins - 1];
                ins--;
            }
            selected[ins] = e;
        }
        for (int route = 0; route < top_k; route++) {
            int e = selected[route];
            uint32_t weight = f2bf(expf(bf2f(logits[e]) - maximum) / denominator);
            out[route] = (weight << 16) | (uint32_t)e;
        }
    }
}

/* sparse_moe_gate_up_fp8_e4m3.comp.template:94-198 + sparse_moe_down_fp8...:90-176
 * + moe_reduce_bf16...:28-45, for all lanes.  gate_up [E][2I][H] e4m3 (I gate
 * rows then I up rows), its scales bf16 [E][ceil(2I/128)][H/128]; down
 * [E][H][I], scales [E][ceil(H/128)][I/128].  Both kernels quantise their bf16
 * input per 128 columns first. */
ORC_API void orc_moe_experts_fp8(const uint16_t *hidden, const uint32_t *routes, const uint8_t *gate_up,
                                 const uint16_t *gate_up_scale, const uint8_t *down, const uint16_t *down_scale,
                                 uint16_t *y, int lanes, int h, int inter, int experts, int top_k, float routed_scale) {
    (void)experts;
    e4m3_init();
    const int block = 128;
    int hb = h / block, ib = inter / block;
    int gu_scale_rows = (2 * inter + block - 1) / block, dn_scale_rows = (h + block - 1) / block;
#pragma omp parallel for
    for (int m = 0; m < lanes; m++) {
        uint8_t *hq = (uint8_t *)malloc(h);
        float *hs = (float *)malloc(sizeof(float) * hb);
        uint16_t *mid = (uint16_t *)malloc(sizeof(uint16_t) * inter);
        uint8_t *mq = (uint8_t *)malloc(inter);
        float *ms = (float *)malloc(sizeof(float) * ib);
        uint16_t *outs = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)top_k * h);
        orc_quantize_fp8(hidden + (size_t)m * h, hq, hs, 1, h, block);
        for (int route = 0; route < top_k; route++) {
            uint32_t word = routes[(size_t)m * top_k + route];
            int e = (int)(word & 0xffffu);
            float route_weight = bf2f((uint16_t)(word >> 16));
            const uint8_t *wgu = gate_up + (size_t)e * 2 * inter * h;
            const uint16_t *sgu = gate_up_scale + (size_t)e * gu_scale_rows * hb;
            for (int row = 0; row < inter; row++) {
                float gate = rbf(dot_fp8(hq, hs, wgu + (size_t)row * h, sgu + (size_t)(row / block) * hb, h, block));
                float up = rbf(dot_fp8(hq, hs, wgu + (size_t)(inter + row) * h,
                                       sgu + (size_t)((inter + row) / block) * hb, h, block));
                mid[row] = f2bf(rbf(rbf(gate / (1.0f + expf(-gate))) * up));
            }
            orc_quantize_fp8(mid, mq, ms, 1, inter, block);
            const uint8_t *wd = down + (size_t)e * h * inter;
            const uint16_t *sd = down_scale + (size_t)e * dn_scale_rows * ib;
            for (int row = 0; row < h; row++) {
                float sum = dot_fp8(mq, ms, wd + (size_t)row * inter, sd + (size_t)(row / block) * ib, inter, block);
                outs[(size_t)route * h + row] = f2bf(rbf(rbf(sum) * route_weight));
            }
        }
        for (int i = 0; i < h; i++) {
            float acc = 0.0f;
            for (int route = 0; route < top_k; route++) acc = rbf(acc + bf2f(outs[(size_t)route * h + i]));
            y[(size_t)m * h + i] = f2bf(acc * routed_scale);
        }
        free(hq);
        free(hs);
        free(mid);
        free(mq);
        free(ms);
        free(outs);
    }
}

/* ---- acceptance: speculative_decode.rs:54-105 ----------------------------- */

/* Returns 0 on success, -1 when the widths disagree (target must be draft+1).
 * out = {accepted, committed}; emitted gets accepted drafts + the target token
 * at the first mismatch; then truncation at the first stop token. */
ORC_API int orc_verify_prefix(const uint32_t *draft, int draft_count, const uint32_t *target, int target_count,
                              const uint32_t *stop, int stop_count, uint32_t *out, uint32_t *emitted,
                              int *emitted_count) {
    if (target_count != draft_count + 1) return -1;
    int accepted = 0;
    while (accepted < draft_count && draft[accepted] == target[accepted]) accepted++;
    int committed = accepted + 1;
    int count = 0;
    for (int i = 0; i < accepted; i++) emitted[count++] = draft[i];
    emitted[count++] = target[accepted];
    for (int i = 0; i < count; i++) {
        int is_stop = 0;
        for (int s = 0; s < stop_count; s++) is_stop |= stop[s] == emitted[i];
        if (is_stop) {
            if (accepted > i + 1) accepted = i + 1;
            committed = i + 1;
            count = i + 1;
            break;
        }
    }
    out[0] = (uint32_t)accepted;
    out[1] = (uint32_t)committed;
    *emitted_count = count;
    return 0;
}

/* ---- kernel-ABI byte layouts the reference's tests pin ----------------------- */

/* stream_control_bytes.rs:8-18: {token u32, tick u64 LE, flags u32, capacity u32} = 20 bytes. */
ORC_API void orc_stream_control_bytes(uint32_t token, uint64_t tick, uint32_t flags, uint32_t capacity, uint8_t *out) {
    uint32_t words[5] = {token, (uint32_t)tick, (uint32_t)(tick >> 32), flags, capacity};
    memcpy(out, words, 20);
}

/* greedy_sampler_f32.comp.template:97-104: the sampler writes the token into word 0 and advances the 64-bit
 * tick held in words 1 (low) and 2 (high). */
ORC_API void orc_sampler_advance_control(uint32_t *control_words, uint32_t token) {
    control_words[0] = token;
    uint32_t next_low = control_words[1] + 1u;
    if (next_low == 0u) control_words[2] += 1u;
    control_words[1] = next_low;
}

/* transient_state_buffer_layout.rs:24-154: header u32[9] = {magic, version, static bytes, static offset,
 * page bytes, page count, dynamic capacity, block capacity, dynamic offset}, then page_table[page_count]
 * (identity), padded to 256 bytes.  Returns the page-table byte capacity; layout_out (if given) receives
 * {block_capacity, page_count, page_bytes, page_table_bytes, static_offset, dynamic_offset, byte_capacity}. */
ORC_API int64_t orc_state_page_table(int64_t static_bytes, int64_t bytes_per_activation, int64_t max_dynamic,
                                     int64_t capacity, uint8_t *table_out, int64_t table_capacity, int64_t *layout_out) {
    const int64_t window = 64, align = 256;
    int64_t dynamic_capacity = 0, block = 0, page_bytes = 0, pages = 0;
    if (bytes_per_activation > 0) {
        if (capacity == 0) return -1;
        dynamic_capacity = max_dynamic > 0 && max_dynamic < capacity ? max_dynamic : capacity;
        block = dynamic_capacity < window ? dynamic_capacity : window;
        page_bytes = bytes_per_activation * block;
        pages = (dynamic_capacity + block - 1) / block;
    }
    if (static_bytes == 0 && pages == 0) return -1;
    int64_t table_bytes = ((9 + pages) * 4 + align - 1) / align * align;
    int64_t static_offset = table_bytes;
    int64_t dynamic_offset = (static_offset + static_bytes + align - 1) / align * align;
    int64_t total = dynamic_offset + page_bytes * pages;
    if (layout_out) {
        int64_t values[7] = {block, pages, page_bytes, table_bytes, static_offset, dynamic_offset, total};
        memcpy(layout_out, values, sizeof(values));
    }
    if (table_out) {
        if (table_capacity < table_bytes) return -1;
        memset(table_out, 0, (size_t)table_bytes);
        uint32_t header[9] = {0x4e525653u, 1u, (uint32_t)static_bytes, (uint32_t)static_offset, (uint32_t)page_bytes,
                              (uint32_t)pages, (uint32_t)dynamic_capacity, (uint32_t)block, (uint32_t)dynamic_offset};
        memcpy(table_out, header, sizeof(header));
        for (int64_t page = 0; page < pages; page++) {
            uint32_t value = (uint32_t)page;
            memcpy(table_out + (9 + page) * 4, &value, 4);
        }
    }
    return table_bytes;
}

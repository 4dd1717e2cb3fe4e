// Element-wise and per-lane kernels: embedding gather, RMSNorm, residual add,
// SiLU*up, concatenate, RoPE (optionally with per-head RMSNorm), FP8 activation
// quantisation, MoE routing and reduce.  All are HBM/L2-trivial (KBs per lane);
// they exist to keep the reference's bf16 rounding points, and are sized so a
// verify batch (<= 160 lanes) fills the SMs with one CTA per lane (x head).
#include "common.cuh"
#include "kernels.cuh"

namespace nerve {

// embedding_lookup_bf16.comp.template:31-46: out = bf16(bf16(row) * scale); a
// token id >= vocab leaves the frame untouched.
__global__ void embedding_kernel(const uint32_t *__restrict__ table, const uint32_t *__restrict__ tokens,
                                 uint32_t *__restrict__ out, int width_words, int vocab, float scale) {
    grid_dependency_wait();
    int lane = blockIdx.y;
    uint32_t token = tokens[lane];
    if (token >= static_cast<uint32_t>(vocab)) return;
    for (int word = blockIdx.x * blockDim.x + threadIdx.x; word < width_words; word += gridDim.x * blockDim.x) {
        uint32_t packed = table[static_cast<size_t>(token) * width_words + word];
        out[static_cast<size_t>(lane) * width_words + word] = pack_bf16(bf16_lo(packed) * scale, bf16_hi(packed) * scale);
    }
}

cudaError_t launch_embedding(const uint16_t *table, const uint32_t *tokens, uint16_t *out, int lanes, int width,
                             int vocab, float scale, cudaStream_t stream) {
    int words = width / 2;
    dim3 grid((words + 255) / 256, lanes);
    embedding_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const uint32_t *>(table), tokens,
                                               reinterpret_cast<uint32_t *>(out), words, vocab, scale);
    return cudaGetLastError();
}

// rms_norm_bf16.comp.template:49-72: y = bf16(x * rsqrt(mean(x^2) + eps) * (w + offset)), f32 math.
__global__ void rms_norm_kernel(const uint32_t *__restrict__ x, const uint32_t *__restrict__ weight,
                                uint32_t *__restrict__ y, int width_words, float inv_width, float eps, float offset) {
    grid_dependency_wait();
    __shared__ float partial[32];
    const uint32_t *row = x + static_cast<size_t>(blockIdx.x) * width_words;
    float sum = 0.0f;
    for (int word = threadIdx.x; word < width_words; word += blockDim.x) {
        uint32_t packed = row[word];
        float lo = bf16_lo(packed), hi = bf16_hi(packed);
        sum = fmaf(lo, lo, sum);
        sum = fmaf(hi, hi, sum);
    }
    sum = warp_sum(sum);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = sum;
    __syncthreads();
    float total = 0.0f;
    for (int warp = 0; warp < (blockDim.x >> 5); warp++) total += partial[warp];
    // IEEE sqrt and divide (nvcc's default -prec-sqrt/-prec-div), as a CPU evaluates 1/sqrt(v)
    float inv_rms = 1.0f / sqrtf(total * inv_width + eps);
    for (int word = threadIdx.x; word < width_words; word += blockDim.x) {
        uint32_t packed = row[word], w = weight[word];
        float lo = bf16_lo(packed) * inv_rms * (bf16_lo(w) + offset);
        float hi = bf16_hi(packed) * inv_rms * (bf16_hi(w) + offset);
        y[static_cast<size_t>(blockIdx.x) * width_words + word] = pack_bf16(lo, hi);
    }
}

cudaError_t launch_rms_norm(const uint16_t *x, const uint16_t *weight, uint16_t *y, int lanes, int width, float eps,
                            float weight_offset, cudaStream_t stream) {
    int words = width / 2;
    int threads = words >= 1024 ? 512 : (words >= 256 ? 256 : (words >= 64 ? 64 : 32));
    rms_norm_kernel<<<lanes, threads, 0, stream>>>(reinterpret_cast<const uint32_t *>(x),
                                                   reinterpret_cast<const uint32_t *>(weight),
                                                   reinterpret_cast<uint32_t *>(y), words, 1.0f / static_cast<float>(width),
                                                   eps, weight_offset);
    return cudaGetLastError();
}

// add_bf16.comp.template:17-24
__global__ void add_kernel(const uint32_t *__restrict__ a, const uint32_t *__restrict__ b, uint32_t *__restrict__ y,
                           size_t words) {
    grid_dependency_wait();
    for (size_t word = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; word < words;
         word += static_cast<size_t>(gridDim.x) * blockDim.x) {
        uint32_t left = a[word], right = b[word];
        y[word] = pack_bf16(bf16_lo(left) + bf16_lo(right), bf16_hi(left) + bf16_hi(right));
    }
}

cudaError_t launch_add(const uint16_t *a, const uint16_t *b, uint16_t *y, size_t count, cudaStream_t stream) {
    size_t words = count / 2;
    int blocks = static_cast<int>((words + 255) / 256);
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (blocks < 1) blocks = 1;
    add_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const uint32_t *>(a), reinterpret_cast<const uint32_t *>(b),
                                           reinterpret_cast<uint32_t *>(y), words);
    return cudaGetLastError();
}

// After the tensor-parallel all-reduce of a row-parallel linear: the reference's linear rounds its f32 sum to bf16
// and its residual_add rounds again (add_bf16.comp.template:17-24).
__global__ void round_add_kernel(const float *__restrict__ sums, const uint16_t *__restrict__ residual, uint16_t *__restrict__ out,
                                 size_t count) {
    for (size_t index = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; index < count;
         index += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float value = round_bf16(sums[index]);
        if (residual != nullptr) value += bf16_bits_to_f32(residual[index]);
        out[index] = static_cast<uint16_t>(f32_to_bf16_bits(value));
    }
}

cudaError_t launch_round_add(const float *sums, const uint16_t *residual, uint16_t *out, size_t count, cudaStream_t stream) {
    int blocks = static_cast<int>((count + 255) / 256);
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (blocks < 1) blocks = 1;
    round_add_kernel<<<blocks, 256, 0, stream>>>(sums, residual, out, count);
    return cudaGetLastError();
}

// silu_multiply_bf16.comp.template:30-52: bf16(bf16(silu(gate)) * up)
__global__ void silu_multiply_kernel(const uint32_t *__restrict__ gate, const uint32_t *__restrict__ up,
                                     uint32_t *__restrict__ y, size_t words) {
    grid_dependency_wait();
    for (size_t word = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; word < words;
         word += static_cast<size_t>(gridDim.x) * blockDim.x) {
        uint32_t g = gate[word], u = up[word];
        y[word] = pack_bf16(rounded_silu(bf16_lo(g)) * bf16_lo(u), rounded_silu(bf16_hi(g)) * bf16_hi(u));
    }
}

cudaError_t launch_silu_multiply(const uint16_t *gate, const uint16_t *up, uint16_t *y, size_t count,
                                 cudaStream_t stream) {
    size_t words = count / 2;
    int blocks = static_cast<int>((words + 255) / 256);
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (blocks < 1) blocks = 1;
    silu_multiply_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const uint32_t *>(gate),
                                                     reinterpret_cast<const uint32_t *>(up),
                                                     reinterpret_cast<uint32_t *>(y), words);
    return cudaGetLastError();
}

// concatenate_bf16.comp.template:20-30 (per lane: [a | b])
__global__ void concat_kernel(const uint32_t *__restrict__ a, const uint32_t *__restrict__ b, uint32_t *__restrict__ y,
                              int words_a, int words_b) {
    grid_dependency_wait();
    int lane = blockIdx.x;
    int total = words_a + words_b;
    for (int word = threadIdx.x; word < total; word += blockDim.x)
        y[static_cast<size_t>(lane) * total + word] =
            word < words_a ? a[static_cast<size_t>(lane) * words_a + word] : b[static_cast<size_t>(lane) * words_b + word - words_a];
}

cudaError_t launch_concat(const uint16_t *a, const uint16_t *b, uint16_t *y, int lanes, int width_a, int width_b,
                          cudaStream_t stream) {
    concat_kernel<<<lanes, 256, 0, stream>>>(reinterpret_cast<const uint32_t *>(a), reinterpret_cast<const uint32_t *>(b),
                                             reinterpret_cast<uint32_t *>(y), width_a / 2, width_b / 2);
    return cudaGetLastError();
}

// rotary_bf16.comp.template:99-109 (five bf16 roundings per element) with
// cos/sin taken from a table the mounter fills with the same f32 pow/cos/sin
// sequence; parallel_head_norm_rope_2way_bf16.comp.template:166-209 when
// norm_weight is given (per-head RMSNorm rounded to bf16 first).
// One CTA per (head, lane); blockDim = head_width/2 rounded up to a warp.
__global__ void rope_kernel(const uint16_t *__restrict__ x, uint16_t *__restrict__ y, const uint32_t *__restrict__ cos_sin,
                            uint32_t table_positions, const uint32_t *__restrict__ positions, int heads, int head_width,
                            int rotary, int interleaved, const uint16_t *__restrict__ norm_weight, float eps, float offset) {
    grid_dependency_wait();
    extern __shared__ float values[];  // head_width normalised (or raw) inputs as f32
    __shared__ float partial[32];
    int head = blockIdx.x, lane = blockIdx.y;
    const uint16_t *in = x + (static_cast<size_t>(lane) * heads + head) * head_width;
    uint16_t *out = y + (static_cast<size_t>(lane) * heads + head) * head_width;
    float sum = 0.0f;
    for (int d = threadIdx.x; d < head_width; d += blockDim.x) {
        float value = bf16_bits_to_f32(in[d]);
        values[d] = value;
        sum = fmaf(value, value, sum);
    }
    if (norm_weight != nullptr) {
        sum = warp_sum(sum);
        if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = sum;
        __syncthreads();
        float total = 0.0f;
        for (int warp = 0; warp < (blockDim.x >> 5); warp++) total += partial[warp];
        float inv_rms = 1.0f / sqrtf(total / static_cast<float>(head_width) + eps);
        for (int d = threadIdx.x; d < head_width; d += blockDim.x)
            values[d] = round_bf16(values[d] * inv_rms * (bf16_bits_to_f32(norm_weight[d]) + offset));
    }
    __syncthreads();
    uint32_t position = positions[lane] % table_positions;
    int half = rotary / 2;
    for (int d = threadIdx.x; d < head_width; d += blockDim.x) {
        float result;
        if (d >= rotary) {
            result = values[d];
        } else {
            int frequency = interleaved ? d / 2 : d % half;
            uint32_t packed = cos_sin[static_cast<size_t>(position) * half + frequency];
            float cosine = bf16_lo(packed), sine = bf16_hi(packed);
            float other;
            if (interleaved) other = (d & 1) == 0 ? -values[d + 1] : values[d - 1];
            else other = d < half ? -values[d + half] : values[d - half];
            float direct = round_bf16(values[d] * cosine);
            float rotated = round_bf16(other * sine);
            result = direct + rotated;
        }
        out[d] = static_cast<uint16_t>(f32_to_bf16_bits(result));
    }
}

cudaError_t launch_rope(const uint16_t *x, uint16_t *y, const uint32_t *cos_sin, uint32_t table_positions,
                        const uint32_t *positions, int lanes, int heads, int head_width, int rotary, int interleaved,
                        const uint16_t *norm_weight, float eps, float weight_offset, cudaStream_t stream) {
    int threads = ((head_width / 2 + 31) / 32) * 32;
    if (threads > 256) threads = 256;
    dim3 grid(heads, lanes);
    rope_kernel<<<grid, threads, head_width * sizeof(float), stream>>>(x, y, cos_sin, table_positions, positions, heads,
                                                                       head_width, rotary, interleaved, norm_weight, eps,
                                                                       weight_offset);
    return cudaGetLastError();
}

// quantize_fp8_e4m3.comp.template:41-60: per 128-column block scale = absmax/448
// (1 when the block is all zero), q = e4m3(x / scale).  One warp per block.
__global__ void quantize_fp8_kernel(const uint32_t *__restrict__ x, uint32_t *__restrict__ q, float *__restrict__ scales,
                                    int blocks_total) {
    grid_dependency_wait();
    int block = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (block >= blocks_total) return;
    int lane = threadIdx.x & 31;
    // 128 columns = 64 words; each thread takes 2 words = 4 values
    const uint32_t *src = x + static_cast<size_t>(block) * 64 + lane * 2;
    uint32_t w0 = src[0], w1 = src[1];
    float v0 = bf16_lo(w0), v1 = bf16_hi(w0), v2 = bf16_lo(w1), v3 = bf16_hi(w1);
    float lane_max = fmaxf(fmaxf(fabsf(v0), fabsf(v1)), fmaxf(fabsf(v2), fabsf(v3)));
    float block_max = warp_max(lane_max);
    float scale = block_max > 0.0f ? block_max / 448.0f : 1.0f;
    if (lane == 0) scales[block] = scale;
    uint32_t packed = static_cast<uint32_t>(f32_to_e4m3(v0 / scale)) | (static_cast<uint32_t>(f32_to_e4m3(v1 / scale)) << 8) |
                      (static_cast<uint32_t>(f32_to_e4m3(v2 / scale)) << 16) |
                      (static_cast<uint32_t>(f32_to_e4m3(v3 / scale)) << 24);
    q[static_cast<size_t>(block) * 32 + lane] = packed;
}

cudaError_t launch_quantize_fp8(const uint16_t *x, uint8_t *q, float *scales, int lanes, int k, cudaStream_t stream) {
    int blocks_total = lanes * (k / 128);
    int warps_per_cta = 8;
    quantize_fp8_kernel<<<(blocks_total + warps_per_cta - 1) / warps_per_cta, warps_per_cta * 32, 0, stream>>>(
        reinterpret_cast<const uint32_t *>(x), reinterpret_cast<uint32_t *>(q), scales, blocks_total);
    return cudaGetLastError();
}

// moe_topk_bf16.comp.template:42-84.  One warp per lane: top_k rounds of
// arg-max (first max wins: lowest expert id among equals), softmax over the
// selected logits accumulated in score order, routes sorted by expert id,
// word = bf16(weight) << 16 | expert.
__global__ void moe_topk_kernel(const uint16_t *__restrict__ router_logits, uint32_t *__restrict__ routes, int experts,
                                int top_k) {
    grid_dependency_wait();
    int token = blockIdx.x;
    int lane = threadIdx.x;
    const uint16_t *logits = router_logits + static_cast<size_t>(token) * experts;
    __shared__ int selected[64];
    __shared__ float selected_score[64];
    for (int route = 0; route < top_k; route++) {
        float best = -INFINITY;
        int best_expert = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            bool taken = false;
            for (int i = 0; i < route; i++) taken |= selected[i] == e;
            float score = bf16_bits_to_f32(logits[e]);
            if (!taken && score > best) {
                best = score;
                best_expert = e;
            }
        }
        for (int offset = 16; offset > 0; offset >>= 1) {
            float other = __shfl_xor_sync(0xffffffffu, best, offset);
            int other_expert = __shfl_xor_sync(0xffffffffu, best_expert, offset);
            if (other > best || (other == best && other_expert < best_expert)) {
                best = other;
                best_expert = other_expert;
            }
        }
        if (best_expert == 0x7fffffff) best_expert = 0;  // every remaining score is -inf or NaN: the shader keeps expert 0
        if (lane == 0) {
            selected[route] = best_expert;
            selected_score[route] = bf16_bits_to_f32(logits[best_expert]);
        }
        __syncwarp();
    }
    if (lane == 0) {
        float maximum = selected_score[0];
        float denominator = 0.0f;
        for (int route = 0; route < top_k; route++) denominator += expf(selected_score[route] - maximum);
        for (int route = 1; route < top_k; route++) {
            int e = selected[route];
            int insertion = route;
            while (insertion > 0 && selected[insertion - 1] > e) {
                selected[insertion] = selected[insertion - 1];
                insertion--;
            }
            selected[insertion] = e;
        }
        for (int route = 0; route < top_k; route++) {
            int e = selected[route];
            uint32_t weight = f32_to_bf16_bits(expf(bf16_bits_to_f32(logits[e]) - maximum) / denominator);
            routes[static_cast<size_t>(token) * top_k + route] = (weight << 16) | static_cast<uint32_t>(e);
        }
    }
}

cudaError_t launch_moe_topk(const uint16_t *router_logits, uint32_t *routes, int lanes, int experts, int top_k,
                            cudaStream_t stream) {
    if (top_k > 64) return cudaErrorInvalidValue;
    moe_topk_kernel<<<lanes, 32, 0, stream>>>(router_logits, routes, experts, top_k);
    return cudaGetLastError();
}

// moe_reduce_bf16.comp.template:28-45: bf16-rounded running sum over the routes
// in route (expert-id) order, then * routed scale.
__global__ void moe_reduce_kernel(const uint32_t *__restrict__ outputs, uint32_t *__restrict__ y, int hidden_words,
                                  int top_k, float routed_scale) {
    grid_dependency_wait();
    int token = blockIdx.x;
    for (int word = threadIdx.x; word < hidden_words; word += blockDim.x) {
        float lo = 0.0f, hi = 0.0f;
        for (int route = 0; route < top_k; route++) {
            uint32_t contribution = outputs[(static_cast<size_t>(token) * top_k + route) * hidden_words + word];
            lo = round_bf16(lo + bf16_lo(contribution));
            hi = round_bf16(hi + bf16_hi(contribution));
        }
        y[static_cast<size_t>(token) * hidden_words + word] = pack_bf16(lo * routed_scale, hi * routed_scale);
    }
}

cudaError_t launch_moe_reduce(const uint16_t *outputs, uint16_t *y, int lanes, int hidden_size, int top_k,
                              float routed_scale, cudaStream_t stream) {
    moe_reduce_kernel<<<lanes, 256, 0, stream>>>(reinterpret_cast<const uint32_t *>(outputs),
                                                 reinterpret_cast<uint32_t *>(y), hidden_size / 2, top_k, routed_scale);
    return cudaGetLastError();
}

}  // namespace nerve

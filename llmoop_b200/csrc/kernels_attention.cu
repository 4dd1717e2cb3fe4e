// Paged-KV GQA attention for decode / verify / prefill-chunk lanes, plus the
// greedy arg-max.  Semantics: append_gqa_attention_bf16.comp.template:189-339
// (each lane's K,V are written at its tick, then it attends over the
// min(tick+1, capacity) most recent tokens; f32 online softmax; one bf16
// rounding at the end).  Because every lane's K,V are appended first and lanes
// of one stream carry increasing ticks, lane i sees exactly the tokens of
// lanes < i plus the committed context - the same result as the reference's
// serial per-lane execution, in one launch.
//
// Work split: one warp per (lane, kv head, context split) serves all
// query heads of that kv head (K/V rows are read once for the group); splits of
// `split_tokens` tokens are merged by a second kernel with a log-sum-exp
// combine.  HBM traffic per launch = the KV bytes of the attended context
// (2 * kv_heads * head_width * 2 B per token) per lane; the scratch partials
// are (head_width + 2) f32 per (lane, q head, split).
#include "common.cuh"
#include "kernels.cuh"

namespace nerve {

__device__ __forceinline__ size_t kv_token_offset(const KvLayer &kv, int slot, uint32_t token, int head, bool value) {
    // token is the ring index (tick % capacity)
    int logical_page = static_cast<int>(token / kv.page_tokens);
    int within = static_cast<int>(token % kv.page_tokens);
    int physical = kv.block_table[static_cast<size_t>(slot) * kv.pages_per_slot + logical_page];
    size_t half = static_cast<size_t>(kv.kv_heads) * kv.page_tokens * kv.head_width;
    return static_cast<size_t>(physical) * (2 * half) + (value ? half : 0) +
           (static_cast<size_t>(head) * kv.page_tokens + within) * kv.head_width;
}

__global__ void kv_append_kernel(const uint32_t *__restrict__ k, const uint32_t *__restrict__ v, KvLayer kv,
                                 LaneTable lanes_meta) {
    grid_dependency_wait();
    int lane = blockIdx.x;
    int slot = lanes_meta.slot[lane];
    if (slot < 0 || kv.capacity == 0) return;
    uint32_t token = lanes_meta.position[lane] % kv.capacity;
    int words_per_head = kv.head_width / 2;
    int total = kv.kv_heads * words_per_head;
    uint32_t *pool = reinterpret_cast<uint32_t *>(kv.pool);
    for (int index = threadIdx.x; index < total; index += blockDim.x) {
        int head = index / words_per_head, word = index % words_per_head;
        size_t k_off = kv_token_offset(kv, slot, token, head, false) / 2 + word;
        size_t v_off = kv_token_offset(kv, slot, token, head, true) / 2 + word;
        pool[k_off] = k[static_cast<size_t>(lane) * total + index];
        pool[v_off] = v[static_cast<size_t>(lane) * total + index];
    }
}

cudaError_t launch_kv_append(const uint16_t *k, const uint16_t *v, const KvLayer &kv, const LaneTable &lanes_meta,
                             int lanes, cudaStream_t stream) {
    if (lanes <= 0) return cudaSuccess;
    kv_append_kernel<<<lanes, 128, 0, stream>>>(reinterpret_cast<const uint32_t *>(k), reinterpret_cast<const uint32_t *>(v),
                                                kv, lanes_meta);
    return cudaGetLastError();
}

size_t attention_scratch_bytes(int lanes, int q_heads, int head_width, int max_splits) {
    return static_cast<size_t>(lanes) * q_heads * max_splits * (head_width + 2) * sizeof(float);
}

// GROUP = query heads per kv head handled by one warp (<= 8), DPL = head dims per thread (head_width / 32).
template <int GROUP, int DPL>
__global__ void __launch_bounds__(128)
attention_split_kernel(const uint16_t *__restrict__ q, KvLayer kv, LaneTable lanes_meta, int lanes, int q_heads,
                       float scale, int split_tokens, int max_splits, float *__restrict__ scratch) {
    constexpr int HD = DPL * 32;
    __shared__ float q_shared[4][GROUP][HD];
    const int warp = threadIdx.x >> 5, lane_id = threadIdx.x & 31;
    const int kv_head = blockIdx.x;
    const int split = blockIdx.y;
    const int lane = blockIdx.z * 4 + warp;
    grid_dependency_wait();
    if (lane >= lanes) return;
    const int slot = lanes_meta.slot[lane];
    if (slot < 0) return;
    const uint32_t tick = lanes_meta.position[lane];
    const uint32_t capacity = kv.capacity;
    const uint32_t tokens = tick + 1u < capacity ? tick + 1u : capacity;
    const uint32_t first_tick = tick + 1u - tokens;  // oldest attended tick
    const uint32_t begin = static_cast<uint32_t>(split) * split_tokens;
    if (begin >= tokens) return;
    const uint32_t end = begin + split_tokens < tokens ? begin + split_tokens : tokens;

    for (int index = lane_id; index < GROUP * HD; index += 32) {
        int head = index / HD, d = index % HD;
        q_shared[warp][head][d] = bf16_bits_to_f32(q[(static_cast<size_t>(lane) * q_heads + kv_head * GROUP + head) * HD + d]);
    }
    __syncwarp();

    float maximum[GROUP], denominator[GROUP], acc[GROUP][DPL];
#pragma unroll
    for (int h = 0; h < GROUP; h++) {
        maximum[h] = -3.4028234663852886e38f;
        denominator[h] = 0.0f;
#pragma unroll
        for (int d = 0; d < DPL; d++) acc[h][d] = 0.0f;
    }

    for (uint32_t chunk = begin; chunk < end; chunk += 32) {
        // each thread scores one token of the chunk against all GROUP query heads
        const uint32_t index = chunk + lane_id;
        const bool valid = index < end;
        float score[GROUP];
#pragma unroll
        for (int h = 0; h < GROUP; h++) score[h] = 0.0f;
        if (valid) {
            uint32_t ring = (first_tick + index) % capacity;
            const uint4 *krow = reinterpret_cast<const uint4 *>(kv.pool + kv_token_offset(kv, slot, ring, kv_head, false));
#pragma unroll 4
            for (int piece = 0; piece < HD / 8; piece++) {
                uint4 kv4 = krow[piece];
                const uint32_t kw[4] = {kv4.x, kv4.y, kv4.z, kv4.w};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    float k0 = bf16_lo(kw[i]), k1 = bf16_hi(kw[i]);
#pragma unroll
                    for (int h = 0; h < GROUP; h++) {
                        score[h] = fmaf(q_shared[warp][h][piece * 8 + 2 * i], k0, score[h]);
                        score[h] = fmaf(q_shared[warp][h][piece * 8 + 2 * i + 1], k1, score[h]);
                    }
                }
            }
        }
        float weight[GROUP];
#pragma unroll
        for (int h = 0; h < GROUP; h++) {
            float s = valid ? score[h] * scale : -3.4028234663852886e38f;
            float chunk_max = warp_max(s);
            float next_max = fmaxf(maximum[h], chunk_max);
            float alpha = expf(maximum[h] - next_max);
            float p = valid ? expf(s - next_max) : 0.0f;
            denominator[h] = denominator[h] * alpha + warp_sum(p);
            maximum[h] = next_max;
            weight[h] = p;
#pragma unroll
            for (int d = 0; d < DPL; d++) acc[h][d] *= alpha;
        }
        // V accumulation: thread owns dims [lane_id*DPL, +DPL); tokens of the chunk in order
        const int count = static_cast<int>(end - chunk < 32u ? end - chunk : 32u);
        for (int t = 0; t < count; t++) {
            uint32_t ring = (first_tick + chunk + t) % capacity;
            const uint16_t *vrow = kv.pool + kv_token_offset(kv, slot, ring, kv_head, true) + lane_id * DPL;
            float vv[DPL];
            if (DPL == 4) {
                uint2 raw = *reinterpret_cast<const uint2 *>(vrow);
                vv[0] = bf16_lo(raw.x);
                vv[1] = bf16_hi(raw.x);
                vv[2 % DPL] = bf16_lo(raw.y);
                vv[3 % DPL] = bf16_hi(raw.y);
            } else if (DPL == 2) {
                uint32_t raw = *reinterpret_cast<const uint32_t *>(vrow);
                vv[0] = bf16_lo(raw);
                vv[1 % DPL] = bf16_hi(raw);
            } else {
#pragma unroll
                for (int d = 0; d < DPL; d++) vv[d] = bf16_bits_to_f32(vrow[d]);
            }
#pragma unroll
            for (int h = 0; h < GROUP; h++) {
                float p = __shfl_sync(0xffffffffu, weight[h], t);
#pragma unroll
                for (int d = 0; d < DPL; d++) acc[h][d] = fmaf(p, vv[d], acc[h][d]);
            }
        }
    }
#pragma unroll
    for (int h = 0; h < GROUP; h++) {
        float *out = scratch + ((static_cast<size_t>(lane) * q_heads + kv_head * GROUP + h) * max_splits + split) * (HD + 2);
#pragma unroll
        for (int d = 0; d < DPL; d++) out[lane_id * DPL + d] = acc[h][d];
        if (lane_id == 0) {
            out[HD] = maximum[h];
            out[HD + 1] = denominator[h];
        }
    }
}

// Small heads (head_width < 32, tiny test models): one thread per (lane, q head), plain loops.
__global__ void attention_small_kernel(const uint16_t *__restrict__ q, uint16_t *__restrict__ out, KvLayer kv,
                                       LaneTable lanes_meta, int lanes, int q_heads, float scale) {
    grid_dependency_wait();
    int index = blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= lanes * q_heads) return;
    int lane = index / q_heads, head = index % q_heads;
    int slot = lanes_meta.slot[lane];
    if (slot < 0) return;
    const int hd = kv.head_width;
    const int kv_head = head / (q_heads / kv.kv_heads);
    const uint32_t tick = lanes_meta.position[lane];
    const uint32_t capacity = kv.capacity;
    const uint32_t tokens = tick + 1u < capacity ? tick + 1u : capacity;
    const uint32_t first_tick = tick + 1u - tokens;
    const uint16_t *qv = q + (static_cast<size_t>(lane) * q_heads + head) * hd;
    float acc[32];
    for (int d = 0; d < hd; d++) acc[d] = 0.0f;
    float maximum = -3.4028234663852886e38f, denominator = 0.0f;
    for (uint32_t i = 0; i < tokens; i++) {
        uint32_t ring = (first_tick + i) % capacity;
        const uint16_t *kr = kv.pool + kv_token_offset(kv, slot, ring, kv_head, false);
        const uint16_t *vr = kv.pool + kv_token_offset(kv, slot, ring, kv_head, true);
        float dot = 0.0f;
        for (int d = 0; d < hd; d++) dot = fmaf(bf16_bits_to_f32(qv[d]), bf16_bits_to_f32(kr[d]), dot);
        float score = dot * scale;
        float next_max = fmaxf(maximum, score);
        float alpha = expf(maximum - next_max), beta = expf(score - next_max);
        denominator = denominator * alpha + beta;
        maximum = next_max;
        for (int d = 0; d < hd; d++) acc[d] = acc[d] * alpha + beta * bf16_bits_to_f32(vr[d]);
    }
    uint16_t *o = out + (static_cast<size_t>(lane) * q_heads + head) * hd;
    for (int d = 0; d < hd; d++) o[d] = static_cast<uint16_t>(f32_to_bf16_bits(denominator == 0.0f ? 0.0f : acc[d] / denominator));
}

// Log-sum-exp merge of the split partials; one warp per (lane, q head).
__global__ void attention_merge_kernel(const float *__restrict__ scratch, uint16_t *__restrict__ out, KvLayer kv,
                                       LaneTable lanes_meta, int lanes, int q_heads, int head_width, int split_tokens,
                                       int max_splits) {
    grid_dependency_wait();
    int pair = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int lane_id = threadIdx.x & 31;
    if (pair >= lanes * q_heads) return;
    int lane = pair / q_heads;
    int slot = lanes_meta.slot[lane];
    if (slot < 0) return;
    uint32_t tick = lanes_meta.position[lane];
    uint32_t tokens = tick + 1u < kv.capacity ? tick + 1u : kv.capacity;
    int splits = static_cast<int>((tokens + split_tokens - 1) / split_tokens);
    if (splits > max_splits) splits = max_splits;
    const float *base = scratch + static_cast<size_t>(pair) * max_splits * (head_width + 2);
    float maximum = -3.4028234663852886e38f;
    for (int s = 0; s < splits; s++) maximum = fmaxf(maximum, base[static_cast<size_t>(s) * (head_width + 2) + head_width]);
    float denominator = 0.0f;
    for (int s = 0; s < splits; s++) {
        const float *part = base + static_cast<size_t>(s) * (head_width + 2);
        denominator += part[head_width + 1] * expf(part[head_width] - maximum);
    }
    for (int d = lane_id; d < head_width; d += 32) {
        float acc = 0.0f;
        for (int s = 0; s < splits; s++) {
            const float *part = base + static_cast<size_t>(s) * (head_width + 2);
            acc += part[d] * expf(part[head_width] - maximum);
        }
        out[static_cast<size_t>(pair) * head_width + d] =
            static_cast<uint16_t>(f32_to_bf16_bits(denominator == 0.0f ? 0.0f : acc / denominator));
    }
}

template <int GROUP>
static cudaError_t launch_split(const uint16_t *q, const KvLayer &kv, const LaneTable &lanes_meta, int lanes, int q_heads,
                                float scale, int split_tokens, int max_splits, float *scratch, cudaStream_t stream) {
    dim3 grid(kv.kv_heads, max_splits, (lanes + 3) / 4);
    switch (kv.head_width) {
    case 128:
        attention_split_kernel<GROUP, 4><<<grid, 128, 0, stream>>>(q, kv, lanes_meta, lanes, q_heads, scale, split_tokens, max_splits, scratch);
        break;
    case 64:
        attention_split_kernel<GROUP, 2><<<grid, 128, 0, stream>>>(q, kv, lanes_meta, lanes, q_heads, scale, split_tokens, max_splits, scratch);
        break;
    case 32:
        attention_split_kernel<GROUP, 1><<<grid, 128, 0, stream>>>(q, kv, lanes_meta, lanes, q_heads, scale, split_tokens, max_splits, scratch);
        break;
    default:
        return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

cudaError_t launch_attention(const uint16_t *q, uint16_t *out, const KvLayer &kv, const LaneTable &lanes_meta,
                             int lanes, int q_heads, float scale, int split_tokens, int max_splits, float *scratch,
                             cudaStream_t stream) {
    if (lanes <= 0) return cudaSuccess;
    const int group = q_heads / kv.kv_heads;
    const bool wide = kv.head_width == 32 || kv.head_width == 64 || kv.head_width == 128;
    if (!wide || (group != 1 && group != 2 && group != 4 && group != 8)) {
        if (kv.head_width > 32) return cudaErrorInvalidValue;
        int total = lanes * q_heads;
        attention_small_kernel<<<(total + 63) / 64, 64, 0, stream>>>(q, out, kv, lanes_meta, lanes, q_heads, scale);
        return cudaGetLastError();
    }
    cudaError_t status;
    switch (group) {
    case 1: status = launch_split<1>(q, kv, lanes_meta, lanes, q_heads, scale, split_tokens, max_splits, scratch, stream); break;
    case 2: status = launch_split<2>(q, kv, lanes_meta, lanes, q_heads, scale, split_tokens, max_splits, scratch, stream); break;
    case 4: status = launch_split<4>(q, kv, lanes_meta, lanes, q_heads, scale, split_tokens, max_splits, scratch, stream); break;
    default: status = launch_split<8>(q, kv, lanes_meta, lanes, q_heads, scale, split_tokens, max_splits, scratch, stream); break;
    }
    if (status != cudaSuccess) return status;
    int pairs = lanes * q_heads;
    attention_merge_kernel<<<(pairs + 3) / 4, 128, 0, stream>>>(scratch, out, kv, lanes_meta, lanes, q_heads, kv.head_width,
                                                                split_tokens, max_splits);
    return cudaGetLastError();
}

// greedy_sampler_f32.comp.template:31-34,52-109: arg-max with ties -> lowest id.  One CTA per lane.
__global__ void argmax_kernel(const float *__restrict__ logits, uint32_t *__restrict__ records, int vocab) {
    grid_dependency_wait();
    __shared__ float best_logit[32];
    __shared__ uint32_t best_token[32];
    const float *row = logits + static_cast<size_t>(blockIdx.x) * vocab;
    float best = -3.4028234663852886e38f;
    uint32_t token = 0xffffffffu;
    for (int index = threadIdx.x; index < vocab; index += blockDim.x) {
        float candidate = row[index];
        if (token == 0xffffffffu || candidate > best) {  // strictly greater keeps the lowest id within a thread
            best = candidate;
            token = static_cast<uint32_t>(index);
        }
    }
    for (int offset = 16; offset > 0; offset >>= 1) {
        float other = __shfl_xor_sync(0xffffffffu, best, offset);
        uint32_t other_token = __shfl_xor_sync(0xffffffffu, token, offset);
        if (other_token != 0xffffffffu && (token == 0xffffffffu || other > best || (other == best && other_token < token))) {
            best = other;
            token = other_token;
        }
    }
    if ((threadIdx.x & 31) == 0) {
        best_logit[threadIdx.x >> 5] = best;
        best_token[threadIdx.x >> 5] = token;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        int warps = blockDim.x >> 5;
        best = threadIdx.x < warps ? best_logit[threadIdx.x] : 0.0f;
        token = threadIdx.x < warps ? best_token[threadIdx.x] : 0xffffffffu;
        for (int offset = 16; offset > 0; offset >>= 1) {
            float other = __shfl_xor_sync(0xffffffffu, best, offset);
            uint32_t other_token = __shfl_xor_sync(0xffffffffu, token, offset);
            if (other_token != 0xffffffffu && (token == 0xffffffffu || other > best || (other == best && other_token < token))) {
                best = other;
                token = other_token;
            }
        }
        if (threadIdx.x == 0) {
            uint32_t *record = records + static_cast<size_t>(blockIdx.x) * 4;
            record[0] = token == 0xffffffffu ? 0u : token;
            record[1] = __float_as_uint(best);
            record[2] = 0u;
            record[3] = 0u;
        }
    }
}

cudaError_t launch_argmax(const float *logits, uint32_t *records, int lanes, int vocab, cudaStream_t stream) {
    if (lanes <= 0) return cudaSuccess;
    argmax_kernel<<<lanes, 1024, 0, stream>>>(logits, records, vocab);
    return cudaGetLastError();
}

}  // namespace nerve

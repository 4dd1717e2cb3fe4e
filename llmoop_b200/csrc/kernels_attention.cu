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

// One CTA (128 threads) serves QL consecutive lanes of one stream x the GROUP query heads of one kv head
// (Q = QL*GROUP query vectors) over one split of the context, tile by tile (TILE tokens):
//   1. the K and V tiles are staged in shared memory with 16-byte loads issued back to back (one exposed
//      latency per tile instead of one per token);
//   2. scores: thread (t = tid % TILE, half = tid / TILE) dots K row t with Q/2 queries (K row stride is padded
//      to HD+8 elements so the 16-byte shared loads of 8 consecutive rows hit distinct banks);
//   3. per-query online softmax over the tile (one warp per query slice), probabilities to shared memory;
//   4. P.V: thread d owns output dims d, d+128, .. for all Q queries, V rows read conflict-free.
// A batch may mix streams: each stream contributes `lanes_per_stream` consecutive lanes, and a CTA never spans
// two streams.
template <int HD, int GROUP, int QL>
__global__ void __launch_bounds__(128)
attention_tile_kernel(const uint16_t *__restrict__ q, KvLayer kv, LaneTable lanes_meta, int lanes, int lanes_per_stream,
                      int q_heads, float scale, int split_tokens, int max_splits, float *__restrict__ scratch) {
    constexpr int TILE = 64;
    constexpr int Q = QL * GROUP;
    constexpr int KSTRIDE = HD + 8;
    constexpr int DPT = HD / 128 > 0 ? HD / 128 : 1;  // output dims per thread (HD = 128 -> 1)
    extern __shared__ __align__(16) uint8_t smem_raw[];
    uint16_t *k_tile = reinterpret_cast<uint16_t *>(smem_raw);                 // [TILE][KSTRIDE]
    uint16_t *v_tile = k_tile + TILE * KSTRIDE;                                 // [TILE][HD]
    uint16_t *q_tile = v_tile + TILE * HD;                                      // [Q][HD]
    float *p_tile = reinterpret_cast<float *>(q_tile + Q * HD);                 // [Q][TILE]
    float *row_max = p_tile + Q * TILE;                                         // [Q]
    float *row_sum = row_max + Q;                                               // [Q]
    float *row_alpha = row_sum + Q;                                             // [Q]
    __shared__ uint32_t lane_tick[QL];

    const int tid = threadIdx.x;
    const int kv_head = blockIdx.x, split = blockIdx.y;
    // lanes of one stream are consecutive and every stream of the batch has `lanes_per_stream` of them
    const int groups_per_stream = (lanes_per_stream + QL - 1) / QL;
    const int stream_index = blockIdx.z / groups_per_stream, group_index = blockIdx.z % groups_per_stream;
    const int lane0 = stream_index * lanes_per_stream + group_index * QL;
    grid_dependency_wait();
    if (lane0 >= lanes) return;
    const int slot = lanes_meta.slot[lane0];
    if (slot < 0) return;
    const uint32_t capacity = kv.capacity;
    // the newest tick among this CTA's lanes bounds the context the CTA has to look at
    uint32_t newest = 0;
    if (tid < QL) {
        int lane = lane0 + tid;
        bool valid = lane < lanes && group_index * QL + tid < lanes_per_stream;
        lane_tick[tid] = valid ? lanes_meta.position[lane] : 0xffffffffu;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < QL; i++)
        if (lane_tick[i] != 0xffffffffu && lane_tick[i] > newest) newest = lane_tick[i];
    const uint32_t tokens = newest + 1u < capacity ? newest + 1u : capacity;  // attended window of the newest lane
    const uint32_t first_tick = newest + 1u - tokens;
    const uint32_t begin = static_cast<uint32_t>(split) * split_tokens;
    if (begin >= tokens) return;
    const uint32_t end = begin + split_tokens < tokens ? begin + split_tokens : tokens;

    for (int index = tid; index < Q * HD / 8; index += 128) {
        int query = index / (HD / 8), piece = index % (HD / 8);
        int lane = lane0 + query / GROUP;
        uint4 value = make_uint4(0, 0, 0, 0);
        if (lane_tick[query / GROUP] != 0xffffffffu)
            value = *reinterpret_cast<const uint4 *>(q + (static_cast<size_t>(lane) * q_heads + kv_head * GROUP + query % GROUP) * HD + piece * 8);
        *reinterpret_cast<uint4 *>(q_tile + query * HD + piece * 8) = value;
    }
    if (tid < Q) {
        row_max[tid] = -3.4028234663852886e38f;
        row_sum[tid] = 0.0f;
    }
    float acc[Q][DPT];
#pragma unroll
    for (int query = 0; query < Q; query++)
#pragma unroll
        for (int d = 0; d < DPT; d++) acc[query][d] = 0.0f;

    for (uint32_t tile_begin = begin; tile_begin < end; tile_begin += TILE) {
        const int count = static_cast<int>(end - tile_begin < TILE ? end - tile_begin : TILE);
        __syncthreads();  // previous tile fully consumed (and q_tile / row_* initialised)
        // ---- stage K and V rows: HD/8 16-byte pieces per row
        for (int index = tid; index < count * (HD / 8); index += 128) {
            int t = index / (HD / 8), piece = index % (HD / 8);
            uint32_t ring = (first_tick + tile_begin + t) % capacity;
            const uint16_t *krow = kv.pool + kv_token_offset(kv, slot, ring, kv_head, false);
            const uint16_t *vrow = kv.pool + kv_token_offset(kv, slot, ring, kv_head, true);
            *reinterpret_cast<uint4 *>(k_tile + t * KSTRIDE + piece * 8) = *reinterpret_cast<const uint4 *>(krow + piece * 8);
            *reinterpret_cast<uint4 *>(v_tile + t * HD + piece * 8) = *reinterpret_cast<const uint4 *>(vrow + piece * 8);
        }
        __syncthreads();
        // ---- scores
        {
            const int t = tid % TILE, half = tid / TILE;
            constexpr int QH = Q / 2 > 0 ? Q / 2 : 1;
            float score[QH];
#pragma unroll
            for (int i = 0; i < QH; i++) score[i] = 0.0f;
            if (t < count && half * QH < Q) {
                for (int piece = 0; piece < HD / 8; piece++) {
                    uint4 kraw = *reinterpret_cast<const uint4 *>(k_tile + t * KSTRIDE + piece * 8);
                    const uint32_t kw[4] = {kraw.x, kraw.y, kraw.z, kraw.w};
#pragma unroll
                    for (int i = 0; i < QH; i++) {
                        uint4 qraw = *reinterpret_cast<const uint4 *>(q_tile + (half * QH + i) * HD + piece * 8);
                        const uint32_t qw[4] = {qraw.x, qraw.y, qraw.z, qraw.w};
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            score[i] = fmaf(bf16_lo(qw[j]), bf16_lo(kw[j]), score[i]);
                            score[i] = fmaf(bf16_hi(qw[j]), bf16_hi(kw[j]), score[i]);
                        }
                    }
                }
            }
            const uint32_t token_tick = first_tick + tile_begin + t;
#pragma unroll
            for (int i = 0; i < QH; i++) {
                int query = half * QH + i;
                if (query >= Q) break;
                uint32_t tick = lane_tick[query / GROUP];
                // causal + ring window of this lane: ticks in (tick - capacity, tick]
                bool visible = t < count && tick != 0xffffffffu && token_tick <= tick && token_tick + capacity > tick;
                p_tile[query * TILE + t] = visible ? score[i] * scale : -INFINITY;
            }
        }
        __syncthreads();
        // ---- online softmax: warp w handles queries w, w+4, ...
        {
            const int warp = tid >> 5, lane_id = tid & 31;
            for (int query = warp; query < Q; query += 4) {
                float s0 = p_tile[query * TILE + lane_id], s1 = p_tile[query * TILE + 32 + lane_id];
                float tile_max = warp_max(fmaxf(s0, s1));
                float old_max = row_max[query];
                float next_max = fmaxf(old_max, tile_max);
                float p0 = 0.0f, p1 = 0.0f, alpha = 1.0f;
                if (next_max > -3.0e38f) {
                    alpha = expf(old_max - next_max);
                    p0 = s0 == -INFINITY ? 0.0f : expf(s0 - next_max);
                    p1 = s1 == -INFINITY ? 0.0f : expf(s1 - next_max);
                }
                float tile_sum = warp_sum(p0 + p1);
                p_tile[query * TILE + lane_id] = p0;
                p_tile[query * TILE + 32 + lane_id] = p1;
                if (lane_id == 0) {
                    row_alpha[query] = alpha;
                    row_sum[query] = row_sum[query] * alpha + tile_sum;
                    row_max[query] = next_max;
                }
            }
        }
        __syncthreads();
        // ---- P.V
#pragma unroll
        for (int query = 0; query < Q; query++) {
            float alpha = row_alpha[query];
#pragma unroll
            for (int d = 0; d < DPT; d++) acc[query][d] *= alpha;
        }
        if (tid < HD || DPT > 1) {
            for (int t = 0; t < count; t++) {
                float vv[DPT];
#pragma unroll
                for (int d = 0; d < DPT; d++) vv[d] = (tid + d * 128 < HD) ? bf16_bits_to_f32(v_tile[t * HD + tid + d * 128]) : 0.0f;
#pragma unroll
                for (int query = 0; query < Q; query++) {
                    float p = p_tile[query * TILE + t];
#pragma unroll
                    for (int d = 0; d < DPT; d++) acc[query][d] = fmaf(p, vv[d], acc[query][d]);
                }
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int query = 0; query < Q; query++) {
        if (lane_tick[query / GROUP] == 0xffffffffu) continue;
        int lane = lane0 + query / GROUP;
        float *out = scratch + ((static_cast<size_t>(lane) * q_heads + kv_head * GROUP + query % GROUP) * max_splits + split) * (HD + 2);
#pragma unroll
        for (int d = 0; d < DPT; d++)
            if (tid + d * 128 < HD) out[tid + d * 128] = acc[query][d];
        if (tid == 0) {
            out[HD] = row_max[query];
            out[HD + 1] = row_sum[query];
        }
    }
}

template <int HD, int GROUP, int QL>
static size_t attention_tile_smem() {
    constexpr int TILE = 64;
    constexpr int Q = QL * GROUP;
    return static_cast<size_t>(TILE) * (HD + 8) * 2 + static_cast<size_t>(TILE) * HD * 2 + static_cast<size_t>(Q) * HD * 2 +
           static_cast<size_t>(Q) * TILE * 4 + 3 * Q * 4;
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

template <int HD, int GROUP, int QL>
static cudaError_t launch_tile(const uint16_t *q, const KvLayer &kv, const LaneTable &lanes_meta, int lanes, int lanes_per_stream,
                               int q_heads, float scale, int split_tokens, int max_splits, float *scratch, cudaStream_t stream) {
    static bool configured = false;
    const size_t smem = attention_tile_smem<HD, GROUP, QL>();
    if (!configured) {
        cudaError_t status = cudaFuncSetAttribute(attention_tile_kernel<HD, GROUP, QL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                  static_cast<int>(smem));
        if (status != cudaSuccess) return status;
        configured = true;
    }
    const int streams = (lanes + lanes_per_stream - 1) / lanes_per_stream;
    dim3 grid(kv.kv_heads, max_splits, streams * ((lanes_per_stream + QL - 1) / QL));
    attention_tile_kernel<HD, GROUP, QL><<<grid, 128, smem, stream>>>(q, kv, lanes_meta, lanes, lanes_per_stream, q_heads, scale, split_tokens,
                                                                      max_splits, scratch);
    return cudaGetLastError();
}

template <int HD>
static cudaError_t launch_tile_group(int group, const uint16_t *q, const KvLayer &kv, const LaneTable &lanes_meta, int lanes,
                                     int lanes_per_stream, int q_heads, float scale, int split_tokens, int max_splits, float *scratch,
                                     cudaStream_t stream) {
    switch (group) {
    case 1: return launch_tile<HD, 1, 4>(q, kv, lanes_meta, lanes, lanes_per_stream, q_heads, scale, split_tokens, max_splits, scratch, stream);
    case 2: return launch_tile<HD, 2, 4>(q, kv, lanes_meta, lanes, lanes_per_stream, q_heads, scale, split_tokens, max_splits, scratch, stream);
    case 4: return launch_tile<HD, 4, 4>(q, kv, lanes_meta, lanes, lanes_per_stream, q_heads, scale, split_tokens, max_splits, scratch, stream);
    case 8: return launch_tile<HD, 8, 2>(q, kv, lanes_meta, lanes, lanes_per_stream, q_heads, scale, split_tokens, max_splits, scratch, stream);
    default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_attention(const uint16_t *q, uint16_t *out, const KvLayer &kv, const LaneTable &lanes_meta,
                             int lanes, int lanes_per_stream, int q_heads, float scale, int split_tokens, int max_splits,
                             float *scratch, cudaStream_t stream) {
    if (lanes <= 0) return cudaSuccess;
    if (lanes_per_stream <= 0 || lanes % lanes_per_stream != 0) return cudaErrorInvalidValue;
    const int group = q_heads / kv.kv_heads;
    const bool wide = kv.head_width == 32 || kv.head_width == 64 || kv.head_width == 128;
    if (!wide || (group != 1 && group != 2 && group != 4 && group != 8)) {
        if (kv.head_width > 32) return cudaErrorInvalidValue;
        int total = lanes * q_heads;
        attention_small_kernel<<<(total + 63) / 64, 64, 0, stream>>>(q, out, kv, lanes_meta, lanes, q_heads, scale);
        return cudaGetLastError();
    }
    cudaError_t status;
    switch (kv.head_width) {
    case 128: status = launch_tile_group<128>(group, q, kv, lanes_meta, lanes, lanes_per_stream, q_heads, scale, split_tokens, max_splits, scratch, stream); break;
    case 64: status = launch_tile_group<64>(group, q, kv, lanes_meta, lanes, lanes_per_stream, q_heads, scale, split_tokens, max_splits, scratch, stream); break;
    default: status = launch_tile_group<32>(group, q, kv, lanes_meta, lanes, lanes_per_stream, q_heads, scale, split_tokens, max_splits, scratch, stream); break;
    }
    if (status != cudaSuccess) return status;
    int pairs = lanes * q_heads;
    attention_merge_kernel<<<(pairs + 3) / 4, 128, 0, stream>>>(scratch, out, kv, lanes_meta, lanes, q_heads, kv.head_width,
                                                                split_tokens, max_splits);
    return cudaGetLastError();
}

// greedy_sampler_f32.comp.template:31-34,52-109: arg-max with ties -> lowest id.  Two stages so that a
// 128k-entry vocabulary is scanned by many CTAs: stage 1 reduces ARGMAX_CHUNKS slices per lane, stage 2 the
// partial winners (chunks are ordered by token id, so "lower id wins a tie" carries over).
constexpr int ARGMAX_CHUNKS = 64;

__device__ __forceinline__ void argmax_combine(float &best, uint32_t &token, float other, uint32_t other_token) {
    if (other_token != 0xffffffffu && (token == 0xffffffffu || other > best || (other == best && other_token < token))) {
        best = other;
        token = other_token;
    }
}

__device__ __forceinline__ void argmax_block_reduce(float &best, uint32_t &token, float *shared_logit, uint32_t *shared_token) {
    for (int offset = 16; offset > 0; offset >>= 1) {
        float other = __shfl_xor_sync(0xffffffffu, best, offset);
        uint32_t other_token = __shfl_xor_sync(0xffffffffu, token, offset);
        argmax_combine(best, token, other, other_token);
    }
    if ((threadIdx.x & 31) == 0) {
        shared_logit[threadIdx.x >> 5] = best;
        shared_token[threadIdx.x >> 5] = token;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        int warps = blockDim.x >> 5;
        best = static_cast<int>(threadIdx.x) < warps ? shared_logit[threadIdx.x] : 0.0f;
        token = static_cast<int>(threadIdx.x) < warps ? shared_token[threadIdx.x] : 0xffffffffu;
        for (int offset = 16; offset > 0; offset >>= 1) {
            float other = __shfl_xor_sync(0xffffffffu, best, offset);
            uint32_t other_token = __shfl_xor_sync(0xffffffffu, token, offset);
            argmax_combine(best, token, other, other_token);
        }
    }
}

__global__ void argmax_partial_kernel(const float *__restrict__ logits, float *__restrict__ partial_logit,
                                      uint32_t *__restrict__ partial_token, int vocab) {
    grid_dependency_wait();
    __shared__ float shared_logit[32];
    __shared__ uint32_t shared_token[32];
    const int lane = blockIdx.y, chunk = blockIdx.x;
    const int per_chunk = (vocab + ARGMAX_CHUNKS - 1) / ARGMAX_CHUNKS;
    const int begin = chunk * per_chunk, end = min(vocab, begin + per_chunk);
    const float *row = logits + static_cast<size_t>(lane) * vocab;
    float best = 0.0f;
    uint32_t token = 0xffffffffu;
    for (int index = begin + threadIdx.x; index < end; index += blockDim.x) {
        float candidate = row[index];
        if (token == 0xffffffffu || candidate > best) {  // strictly greater keeps the lowest id within a thread
            best = candidate;
            token = static_cast<uint32_t>(index);
        }
    }
    argmax_block_reduce(best, token, shared_logit, shared_token);
    if (threadIdx.x == 0) {
        partial_logit[lane * ARGMAX_CHUNKS + chunk] = best;
        partial_token[lane * ARGMAX_CHUNKS + chunk] = token;
    }
}

__global__ void argmax_final_kernel(const float *__restrict__ partial_logit, const uint32_t *__restrict__ partial_token,
                                    uint32_t *__restrict__ records) {
    grid_dependency_wait();
    __shared__ float shared_logit[32];
    __shared__ uint32_t shared_token[32];
    const int lane = blockIdx.x;
    float best = partial_logit[lane * ARGMAX_CHUNKS + threadIdx.x];
    uint32_t token = partial_token[lane * ARGMAX_CHUNKS + threadIdx.x];
    argmax_block_reduce(best, token, shared_logit, shared_token);
    if (threadIdx.x == 0) {
        uint32_t *record = records + static_cast<size_t>(lane) * 4;
        record[0] = token == 0xffffffffu ? 0u : token;
        record[1] = __float_as_uint(best);
        record[2] = 0u;
        record[3] = 0u;
    }
}

size_t argmax_scratch_bytes(int lanes) { return static_cast<size_t>(lanes) * ARGMAX_CHUNKS * 8; }

cudaError_t launch_argmax(const float *logits, uint32_t *records, int lanes, int vocab, void *scratch, cudaStream_t stream) {
    if (lanes <= 0) return cudaSuccess;
    float *partial_logit = static_cast<float *>(scratch);
    uint32_t *partial_token = reinterpret_cast<uint32_t *>(partial_logit + static_cast<size_t>(lanes) * ARGMAX_CHUNKS);
    dim3 grid(ARGMAX_CHUNKS, lanes);
    argmax_partial_kernel<<<grid, 256, 0, stream>>>(logits, partial_logit, partial_token, vocab);
    cudaError_t status = cudaGetLastError();
    if (status != cudaSuccess) return status;
    argmax_final_kernel<<<lanes, ARGMAX_CHUNKS, 0, stream>>>(partial_logit, partial_token, records);
    return cudaGetLastError();
}

}  // namespace nerve

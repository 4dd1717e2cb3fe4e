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
#include <atomic>

#include "attention_body.cuh"
#include "common.cuh"
#include "kernels.cuh"

namespace nerve {

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

// One CTA (128 threads) = one team of attention_tile_body (attention_body.cuh): grid (kv head, split, stream x lane group).
template <int HD, int GROUP, int QL>
__global__ void __launch_bounds__(128)
attention_tile_kernel(const uint16_t *__restrict__ q, KvLayer kv, LaneTable lanes_meta, int lanes, int lanes_per_stream,
                      int q_heads, float scale, int split_tokens, int max_splits, float *__restrict__ scratch) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    grid_dependency_wait();
    attention_tile_body<HD, GROUP, QL, false>(q, kv, lanes_meta, lanes, lanes_per_stream, q_heads, scale, split_tokens, max_splits,
                                              scratch, blockIdx.x, blockIdx.y, blockIdx.z, smem_raw, threadIdx.x, 0);
}

template <int HD, int GROUP, int QL>
static size_t attention_tile_smem() {
    return attention_team_smem<HD, GROUP, QL>();
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
    if (pair >= lanes * q_heads) return;
    attention_merge_pair<false>(scratch, out, kv, lanes_meta, pair, threadIdx.x & 31, q_heads, head_width, split_tokens, max_splits);
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

// ---- greedy arg-max without a caller-provided scratch buffer -------------------------------------------------
// Same two kernels as launch_argmax, with the per-chunk partial winners kept in a fixed device array that is part
// of the library image (32 KB, enough for STATIC_ARGMAX_MAX_LANES lanes).  Nothing is allocated, by this function
// or on its behalf: the array's device address is looked up once per device (cudaGetSymbolAddress; the array's
// name on the host side is not a device pointer) with that device current, and cached.
// Every partial slot the second kernel reads is written by the first kernel of the same call, so nothing needs
// clearing between calls; the array does keep the previous call's partials and is shared by all callers in the
// process, so two calls that overlap in time on one device (different streams or threads) race on it.
constexpr int STATIC_ARGMAX_MAX_LANES = 64;
constexpr int STATIC_ARGMAX_MAX_DEVICES = 64;
static __device__ __align__(256) unsigned char static_argmax_scratch[STATIC_ARGMAX_MAX_LANES * ARGMAX_CHUNKS * 8];

int argmax_static_max_lanes() { return STATIC_ARGMAX_MAX_LANES; }

cudaError_t launch_argmax_static(const float *logits, uint32_t *records, int lanes, int vocab, cudaStream_t stream) {
    if (lanes <= 0) return cudaSuccess;
    if (lanes > STATIC_ARGMAX_MAX_LANES) return cudaErrorInvalidValue;
    static std::atomic<void *> device_address[STATIC_ARGMAX_MAX_DEVICES];  // zero-initialised; every thread that looks it up stores the same value
    int device = 0;
    cudaError_t status = cudaGetDevice(&device);
    if (status != cudaSuccess) return status;
    if (device < 0 || device >= STATIC_ARGMAX_MAX_DEVICES) return cudaErrorInvalidDevice;
    void *address = device_address[device].load(std::memory_order_acquire);
    if (address == nullptr) {
        status = cudaGetSymbolAddress(&address, static_argmax_scratch);
        if (status != cudaSuccess) return status;
        device_address[device].store(address, std::memory_order_release);
    }
    return launch_argmax(logits, records, lanes, vocab, address, stream);
}

}  // namespace nerve

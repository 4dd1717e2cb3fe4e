// Seeded temperature / top-k / top-p / min-p sampler (sampler.rs:748-873), per lane, from f32 logits:
//   temperature_top_k_candidates_f32.comp.template:48-127  exact sorted top-k of each vocabulary partition
//   temperature_top_k_top_p_sampler_f32.comp.template:56-72,100-216  merge, weights, nucleus, seeded draw
// Stage 1: one CTA per (lane, vocabulary chunk) stages its chunk in shared memory and extracts its exact top-k
// (larger logit first, ties -> lower id, NaNs skipped) by k block-wide arg-max passes.  Stage 2: one CTA per lane
// merges the chunk lists into the global top-k and one thread does the shader's serial f32 arithmetic in list
// order: max_scaled = top0/T, min-p cut, total weight, top-p nucleus, u = (hash(seed ^ tick) >> 8) * 2^-24, pick
// the first index whose cumulative weight exceeds u * nucleus weight.  A lane whose stream is greedy (method 0)
// takes the first entry and writes flags 0, so one launch serves mixed batches.
// record = {token, logit bits, 1 (sampled) or 0 (greedy), 0}.
#include "common.cuh"
#include "kernels.cuh"

namespace nerve {

namespace {

constexpr int SAMPLE_CHUNKS = 64;
constexpr int SAMPLE_THREADS = 256;
constexpr float LOWEST = -3.4028234663852886e38f;

__device__ __forceinline__ bool better(float logit, uint32_t token, float other_logit, uint32_t other_token) {
    return logit > other_logit || (logit == other_logit && token < other_token);
}

__device__ __forceinline__ uint32_t hash_u32(uint32_t value) {
    value ^= value >> 16;
    value *= 0x7feb352du;
    value ^= value >> 15;
    value *= 0x846ca68bu;
    value ^= value >> 16;
    return value;
}

// Block-wide best (logit desc, token asc) of one candidate per thread; every thread returns the winner.
__device__ __forceinline__ void block_best(float &logit, uint32_t &token, float *shared_logit, uint32_t *shared_token) {
    for (int offset = 16; offset > 0; offset >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, logit, offset);
        const uint32_t other_token = __shfl_xor_sync(0xffffffffu, token, offset);
        if (better(other, other_token, logit, token)) {
            logit = other;
            token = other_token;
        }
    }
    const int warps = blockDim.x >> 5;
    __syncthreads();  // the previous pass's winners have been read
    if ((threadIdx.x & 31) == 0) {
        shared_logit[threadIdx.x >> 5] = logit;
        shared_token[threadIdx.x >> 5] = token;
    }
    __syncthreads();
    logit = shared_logit[0];
    token = shared_token[0];
    for (int w = 1; w < warps; w++)
        if (better(shared_logit[w], shared_token[w], logit, token)) {
            logit = shared_logit[w];
            token = shared_token[w];
        }
}

__device__ __forceinline__ SamplerParams params_of(const SamplerParams *table, const int32_t *slots, int lane) {
    const int slot = slots != nullptr ? slots[lane] : 0;
    SamplerParams params = table[slot < 0 ? 0 : slot];
    if (params.method == 0 || params.top_k < 1) params.top_k = 1;
    if (params.top_k > SAMPLER_MAX_TOP_K) params.top_k = SAMPLER_MAX_TOP_K;
    return params;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_candidates_kernel(const float *__restrict__ logits, uint2 *__restrict__ candidates, const SamplerParams *__restrict__ table,
                         const int32_t *__restrict__ slots, int vocab) {
    extern __shared__ float chunk_values[];
    __shared__ float shared_logit[SAMPLE_THREADS / 32];
    __shared__ uint32_t shared_token[SAMPLE_THREADS / 32];
    const int lane = blockIdx.y, chunk = blockIdx.x;
    const int per_chunk = (vocab + SAMPLE_CHUNKS - 1) / SAMPLE_CHUNKS;
    const int begin = chunk * per_chunk, end = min(vocab, begin + per_chunk);
    const int top_k = params_of(table, slots, lane).top_k;
    const float *row = logits + static_cast<size_t>(lane) * vocab;
    for (int index = begin + threadIdx.x; index < end; index += blockDim.x) chunk_values[index - begin] = row[index];
    __syncthreads();
    float previous_logit = 0.0f;
    uint32_t previous_token = 0;
    uint2 *out = candidates + (static_cast<size_t>(lane) * SAMPLE_CHUNKS + chunk) * SAMPLER_MAX_TOP_K;
    for (int rank = 0; rank < top_k; rank++) {
        float best = LOWEST;
        uint32_t best_token = 0xffffffffu;
        for (int index = begin + threadIdx.x; index < end; index += blockDim.x) {
            const float candidate = chunk_values[index - begin];
            const uint32_t token = static_cast<uint32_t>(index);
            if (isnan(candidate)) continue;
            // after the first pass only entries that come after the previous winner in the order still count
            if (rank != 0 && !(candidate < previous_logit || (candidate == previous_logit && token > previous_token))) continue;
            if (better(candidate, token, best, best_token)) {
                best = candidate;
                best_token = token;
            }
        }
        block_best(best, best_token, shared_logit, shared_token);
        if (threadIdx.x == 0) out[rank] = make_uint2(__float_as_uint(best), best_token);
        previous_logit = best;
        previous_token = best_token;
    }
}

__global__ void __launch_bounds__(SAMPLE_CHUNKS)
sample_draw_kernel(const uint2 *__restrict__ candidates, uint32_t *__restrict__ records, const SamplerParams *__restrict__ table,
                   const int32_t *__restrict__ slots, const uint32_t *__restrict__ ticks) {
    __shared__ float shared_logit[SAMPLE_CHUNKS / 32];
    __shared__ uint32_t shared_token[SAMPLE_CHUNKS / 32];
    __shared__ float top_logit[SAMPLER_MAX_TOP_K];
    __shared__ uint32_t top_token[SAMPLER_MAX_TOP_K];
    const int lane = blockIdx.x;
    const SamplerParams params = params_of(table, slots, lane);
    const uint2 *mine = candidates + (static_cast<size_t>(lane) * SAMPLE_CHUNKS + threadIdx.x) * SAMPLER_MAX_TOP_K;
    int cursor = 0;
    for (int rank = 0; rank < params.top_k; rank++) {
        const uint2 head = mine[cursor];
        float logit = __uint_as_float(head.x);
        uint32_t token = head.y;
        const uint32_t offered = token;
        block_best(logit, token, shared_logit, shared_token);
        if (threadIdx.x == 0) {
            top_logit[rank] = logit;
            top_token[rank] = token;
        }
        // the chunk whose head won moves on (token ids are unique across chunks; an exhausted list offers 0xffffffff)
        if (offered == token && token != 0xffffffffu && cursor + 1 < SAMPLER_MAX_TOP_K) cursor++;
    }
    __syncthreads();
    if (threadIdx.x != 0) return;
    uint32_t *record = records + static_cast<size_t>(lane) * 4;
    int selected = 0;
    if (params.method != 0) {
        const float temperature = params.temperature;
        const float max_scaled = top_logit[0] / temperature;
        const float min_logit = params.min_p > 0.0f ? top_logit[0] + temperature * logf(params.min_p) : LOWEST;
        float total = 0.0f;
        for (int i = 0; i < params.top_k; i++) {
            if (top_logit[i] < min_logit) break;
            total += expf(top_logit[i] / temperature - max_scaled);
        }
        const float threshold = params.top_p * total;
        float nucleus = 0.0f;
        int count = 0;
        for (int i = 0; i < params.top_k; i++) {
            if (top_logit[i] < min_logit) break;
            nucleus += expf(top_logit[i] / temperature - max_scaled);
            count = i + 1;
            if (nucleus >= threshold) break;
        }
        const uint32_t tick_low = ticks != nullptr ? ticks[lane] : 0u;
        const uint32_t bits = hash_u32(params.seed ^ tick_low);  // the lanes' ticks are 32-bit here: high word 0
        const float target = static_cast<float>(bits >> 8) * (1.0f / 16777216.0f) * nucleus;
        float cumulative = 0.0f;
        selected = count > 0 ? count - 1 : 0;
        for (int i = 0; i < count; i++) {
            cumulative += expf(top_logit[i] / temperature - max_scaled);
            if (target < cumulative) {
                selected = i;
                break;
            }
        }
    }
    const uint32_t token = top_token[selected];
    record[0] = token == 0xffffffffu ? 0u : token;
    record[1] = __float_as_uint(top_logit[selected]);
    record[2] = params.method != 0 ? 1u : 0u;
    record[3] = 0u;
}

}  // namespace

size_t sampler_scratch_bytes(int lanes) { return static_cast<size_t>(lanes) * SAMPLE_CHUNKS * SAMPLER_MAX_TOP_K * sizeof(uint2); }

cudaError_t launch_sample(const float *logits, uint32_t *records, int lanes, int vocab, const SamplerParams *table, const int32_t *slots,
                          const uint32_t *ticks, void *scratch, cudaStream_t stream) {
    if (lanes <= 0) return cudaSuccess;
    if (vocab <= 0 || table == nullptr || scratch == nullptr) return cudaErrorInvalidValue;
    const int per_chunk = (vocab + SAMPLE_CHUNKS - 1) / SAMPLE_CHUNKS;
    const size_t smem = static_cast<size_t>(per_chunk) * sizeof(float);
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        cudaError_t status = cudaFuncSetAttribute(sample_candidates_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (status != cudaSuccess) return status;
        configured = true;
    }
    uint2 *candidates = static_cast<uint2 *>(scratch);
    sample_candidates_kernel<<<dim3(SAMPLE_CHUNKS, lanes), SAMPLE_THREADS, smem, stream>>>(logits, candidates, table, slots, vocab);
    cudaError_t status = cudaGetLastError();
    if (status != cudaSuccess) return status;
    sample_draw_kernel<<<lanes, SAMPLE_CHUNKS, 0, stream>>>(candidates, records, table, slots, ticks);
    return cudaGetLastError();
}

}  // namespace nerve

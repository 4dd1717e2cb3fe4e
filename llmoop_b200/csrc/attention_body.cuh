// Device-side bodies of the paged-KV attention (one context split of one kv head for up to QL lanes of a
// stream) and of the split merge, shared by the stand-alone attention kernels and by the persistent decode
// stack kernel.  A body is run by a team of 128 threads that synchronises on a named barrier, so four teams can
// work side by side inside one 512-thread CTA.
// Semantics: append_gqa_attention_bf16.comp.template:189-339 (f32 online softmax, one bf16 rounding at the end).
#pragma once

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

__device__ __forceinline__ void team_sync(int barrier_id) { asm volatile("bar.sync %0, 128;" ::"r"(barrier_id) : "memory"); }

// COHERENT: the query vectors were written by other CTAs of the same launch and are read through L2.
template <bool COHERENT>
__device__ __forceinline__ uint4 load_activation16(const void *address) {
    return COHERENT ? __ldcg(reinterpret_cast<const uint4 *>(address)) : *reinterpret_cast<const uint4 *>(address);
}

template <int HD, int GROUP, int QL>
__host__ __device__ constexpr size_t attention_team_smem() {
    constexpr int TILE = 64;
    constexpr int Q = QL * GROUP;
    // K tile (padded rows), V tile, Q tile, probabilities, three per-query rows, the lanes' ticks
    return static_cast<size_t>(TILE) * (HD + 8) * 2 + static_cast<size_t>(TILE) * HD * 2 + static_cast<size_t>(Q) * HD * 2 +
           static_cast<size_t>(Q) * TILE * 4 + 3 * Q * 4 + ((QL * 4 + 15) / 16) * 16;
}

// The team serves QL consecutive lanes of one stream x the GROUP query heads of one kv head (Q = QL*GROUP query
// vectors) over one split of the context, tile by tile (TILE tokens):
//   1. the K and V tiles are staged in shared memory with 16-byte loads issued back to back (one exposed
//      latency per tile instead of one per token);
//   2. scores: thread (t = tid % TILE, half = tid / TILE) dots K row t with Q/2 queries (K row stride is padded
//      to HD+8 elements so the 16-byte shared loads of 8 consecutive rows hit distinct banks);
//   3. per-query online softmax over the tile (one warp per query slice), probabilities to shared memory;
//   4. P.V: thread d owns output dims d, d+128, .. for all Q queries, V rows read conflict-free.
// A batch may mix streams: each stream contributes `lanes_per_stream` consecutive lanes, and a team never spans
// two streams.  `group_slot` enumerates (stream, lane group) pairs.
template <int HD, int GROUP, int QL, bool COHERENT>
__device__ void attention_tile_body(const uint16_t *__restrict__ q, const KvLayer &kv, const LaneTable &lanes_meta, int lanes,
                                    int lanes_per_stream, int q_heads, float scale, int split_tokens, int max_splits,
                                    float *__restrict__ scratch, int kv_head, int split, int group_slot, uint8_t *smem_raw,
                                    int tid, int barrier_id) {
    constexpr int TILE = 64;
    constexpr int Q = QL * GROUP;
    constexpr int KSTRIDE = HD + 8;
    constexpr int DPT = HD / 128 > 0 ? HD / 128 : 1;  // output dims per thread (HD = 128 -> 1)
    uint16_t *k_tile = reinterpret_cast<uint16_t *>(smem_raw);                 // [TILE][KSTRIDE]
    uint16_t *v_tile = k_tile + TILE * KSTRIDE;                                 // [TILE][HD]
    uint16_t *q_tile = v_tile + TILE * HD;                                      // [Q][HD]
    float *p_tile = reinterpret_cast<float *>(q_tile + Q * HD);                 // [Q][TILE]
    float *row_max = p_tile + Q * TILE;                                         // [Q]
    float *row_sum = row_max + Q;                                               // [Q]
    float *row_alpha = row_sum + Q;                                             // [Q]
    uint32_t *lane_tick = reinterpret_cast<uint32_t *>(row_alpha + Q);          // [QL]

    // lanes of one stream are consecutive and every stream of the batch has `lanes_per_stream` of them
    const int groups_per_stream = (lanes_per_stream + QL - 1) / QL;
    const int stream_index = group_slot / groups_per_stream, group_index = group_slot % groups_per_stream;
    const int lane0 = stream_index * lanes_per_stream + group_index * QL;
    if (lane0 >= lanes) return;
    const int slot = lanes_meta.slot[lane0];
    if (slot < 0) return;
    const uint32_t capacity = kv.capacity;
    team_sync(barrier_id);  // the previous item of this team no longer reads the shared arrays
    // the newest tick among this team's lanes bounds the context the team has to look at
    uint32_t newest = 0;
    if (tid < QL) {
        int lane = lane0 + tid;
        bool valid = lane < lanes && group_index * QL + tid < lanes_per_stream;
        lane_tick[tid] = valid ? lanes_meta.position[lane] : 0xffffffffu;
    }
    team_sync(barrier_id);
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
            value = load_activation16<COHERENT>(q + (static_cast<size_t>(lane) * q_heads + kv_head * GROUP + query % GROUP) * HD + piece * 8);
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
        team_sync(barrier_id);  // previous tile fully consumed (and q_tile / row_* initialised)
        // ---- stage K and V rows: HD/8 16-byte pieces per row
        for (int index = tid; index < count * (HD / 8); index += 128) {
            int t = index / (HD / 8), piece = index % (HD / 8);
            uint32_t ring = (first_tick + tile_begin + t) % capacity;
            const uint16_t *krow = kv.pool + kv_token_offset(kv, slot, ring, kv_head, false);
            const uint16_t *vrow = kv.pool + kv_token_offset(kv, slot, ring, kv_head, true);
            *reinterpret_cast<uint4 *>(k_tile + t * KSTRIDE + piece * 8) = load_activation16<COHERENT>(krow + piece * 8);
            *reinterpret_cast<uint4 *>(v_tile + t * HD + piece * 8) = load_activation16<COHERENT>(vrow + piece * 8);
        }
        team_sync(barrier_id);
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
        team_sync(barrier_id);
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
        team_sync(barrier_id);
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
    team_sync(barrier_id);
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

// Log-sum-exp merge of the split partials of one (lane, q head) pair by one warp.
template <bool COHERENT>
__device__ __forceinline__ void attention_merge_pair(const float *__restrict__ scratch, uint16_t *__restrict__ out, const KvLayer &kv,
                                                     const LaneTable &lanes_meta, int pair, int lane_id, int q_heads, int head_width,
                                                     int split_tokens, int max_splits) {
    int lane = pair / q_heads;
    int slot = lanes_meta.slot[lane];
    if (slot < 0) return;
    uint32_t tick = lanes_meta.position[lane];
    uint32_t tokens = tick + 1u < kv.capacity ? tick + 1u : kv.capacity;
    int splits = static_cast<int>((tokens + split_tokens - 1) / split_tokens);
    if (splits > max_splits) splits = max_splits;
    const float *base = scratch + static_cast<size_t>(pair) * max_splits * (head_width + 2);
    auto read = [&](const float *address) { return COHERENT ? __ldcg(address) : *address; };
    float maximum = -3.4028234663852886e38f;
    for (int s = 0; s < splits; s++) maximum = fmaxf(maximum, read(base + static_cast<size_t>(s) * (head_width + 2) + head_width));
    float denominator = 0.0f;
    for (int s = 0; s < splits; s++) {
        const float *part = base + static_cast<size_t>(s) * (head_width + 2);
        denominator += read(part + head_width + 1) * expf(read(part + head_width) - maximum);
    }
    for (int d = lane_id; d < head_width; d += 32) {
        float acc = 0.0f;
        for (int s = 0; s < splits; s++) {
            const float *part = base + static_cast<size_t>(s) * (head_width + 2);
            acc += read(part + d) * expf(read(part + head_width) - maximum);
        }
        out[static_cast<size_t>(pair) * head_width + d] =
            static_cast<uint16_t>(f32_to_bf16_bits(denominator == 0.0f ? 0.0f : acc / denominator));
    }
}

}  // namespace nerve

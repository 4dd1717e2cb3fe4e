// Persistent decode stack: one cooperative launch runs every layer of a dense INT4 g128 Llama-style stack
// (rms_norm, q/k/v, RoPE, KV append, attention, o + residual, rms_norm, gate/up + SiLU, down + residual:
// the kernel list of one reference layer component, runtime-rs/shaders/*.comp.template) for a batch of at most
// 8 lanes - the verify batch and the draft / single-tick steps of the speculative decode cycle.
//
// Why one launch: at these batch sizes a layer is ~136 MB of weights (~21 us of HBM time) cut into a dozen
// dependent steps; as separate kernels every step pays a launch, a pipeline fill and a drain (~6 us each,
// measured), which is several times the streaming time.  Here one CTA per SM stays resident, keeps a register
// ring of packed weights in flight across step boundaries (weights do not depend on activations, so the next
// matrix is already streaming while the grid waits at a barrier), and the steps are separated by grid-wide
// barriers (bounded spins on one global counter).
//
// Data layout:
//  * weights: a tile-major copy made at mount - [tile of 16 rows][group of 128 columns][rt][half][lane] uint4,
//    i.e. exactly the order in which a warp's two 16-byte loads consume them (each load is 512 contiguous
//    bytes; a tile is K/128 contiguous KB).  q and k tiles pair row d with row d + head_width/2, so RoPE runs in
//    the q/k/v epilogue and K, V go straight into the KV pages.
//  * activations of a step: staged once per CTA in shared memory in mma.sync B-fragment order, together with
//    136 * sum(x) per (lane, group): the nibbles are fed to the tensor cores as bf16 128+q (one lop3 per pair,
//    no subtract) and the bias 128+8 is taken out per group with that sum.
//  * a matrix tile is computed by all 16 warps of a CTA (each takes every 16th group of K), reduced through
//    shared memory, and finished by 64 epilogue threads.
#include "attention_body.cuh"
#include "common.cuh"
#include "kernels.cuh"

namespace nerve {

namespace {

constexpr int STACK_WARPS = 16;
constexpr int STACK_THREADS = STACK_WARPS * 32;
constexpr int RING_UNITS = 4;          // 16x128 weight blocks a warp keeps in flight
constexpr int ATTENTION_TEAMS = 4;     // 128-thread teams per CTA in the attention phase
constexpr int ATTENTION_QL = 4;        // lanes of one stream served by one team
constexpr unsigned int BARRIER_SPIN_LIMIT = 1u << 20;

// ------------------------------------------------------------------------------------------ tile-major copy

struct RelayoutArgs {
    RelayoutSegment segment[3];
    int first_tile[4];
    int count;
    int pair;
    int k;
    int tiles;
};

__global__ void int4_tile_major_kernel(const RelayoutArgs args, uint4 *__restrict__ weights_out, uint32_t *__restrict__ scales_out) {
    const int groups = args.k >> 7, rt_count = args.pair ? 2 : 1;
    const size_t total = static_cast<size_t>(args.tiles) * groups * rt_count * 64;
    for (size_t index = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; index < total;
         index += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int lane = static_cast<int>(index & 31), half = static_cast<int>((index >> 5) & 1);
        size_t rest = index >> 6;
        const int rt = static_cast<int>(rest % rt_count);
        rest /= rt_count;
        const int group = static_cast<int>(rest % groups), tile = static_cast<int>(rest / groups);
        const int g = lane >> 2, j = lane & 3;
        int which = 0, local_tile = tile;
        if (args.pair) {
            which = rt;
        } else {
            while (which + 1 < args.count && tile >= args.first_tile[which + 1]) which++;
            local_tile = tile - args.first_tile[which];
        }
        const RelayoutSegment &segment = args.segment[which];
        auto source_row = [&](int mma_row) {
            if (segment.rope_head_width > 0) {
                const int tiles_per_head = segment.rope_head_width / 16;
                const int head = local_tile / tiles_per_head, th = local_tile % tiles_per_head;
                const int d = mma_row < 8 ? 8 * th + mma_row : segment.rope_head_width / 2 + 8 * th + (mma_row - 8);
                return head * segment.rope_head_width + d;
            }
            return local_tile * 16 + mma_row;
        };
        const int row = source_row(g + 8 * half);
        weights_out[index] = *reinterpret_cast<const uint4 *>(segment.qweight + static_cast<size_t>(row) * (args.k >> 3) + group * 16 + j * 4);
        if (half == 0 && j == 0) {
            const uint32_t low = segment.scales[static_cast<size_t>(row) * groups + group];
            const uint32_t high = segment.scales[static_cast<size_t>(source_row(g + 8)) * groups + group];
            scales_out[(static_cast<size_t>(tile) * groups + group) * rt_count * 8 + rt * 8 + g] = low | (high << 16);
        }
    }
}

// ------------------------------------------------------------------------------------------ small helpers

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Nibbles at bits s..s+3 and s+16..s+19 of `word` -> bf16x2 (128 + q, 128 + q'): 0x4300 | q is exactly 128 + q.
__device__ __forceinline__ uint32_t biased_pair(uint32_t word, int shift) {
    uint32_t out;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(out) : "r"(word >> shift), "n"(0x000F000F), "n"(0x43004300));
    return out;
}

__device__ __forceinline__ uint32_t load_acquire(const unsigned int *address) {
    uint32_t value;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(value) : "l"(address) : "memory");
    return value;
}

// All CTAs of the (cooperative, co-resident) grid meet here.  `target` counts the arrivals expected so far.  A
// wait that does not complete within the spin limit sets the error flag and lets the CTA go on (its results are
// then garbage, the host sees the flag); once the flag is up nobody waits any more.
__device__ __forceinline__ void grid_barrier(unsigned int *counter, unsigned int &target, int *error_flag) {
    __syncthreads();
    if (threadIdx.x == 0) {
        target += gridDim.x;
        __threadfence();
        atomicAdd(counter, 1u);
        unsigned int spins = 0;
        while (load_acquire(counter) < target) {
            if (++spins > BARRIER_SPIN_LIMIT) {
                atomicExch(error_flag, 2);
                break;
            }
            if ((spins & 63u) == 0 && *reinterpret_cast<volatile int *>(error_flag) != 0) break;
            __nanosleep(32);
        }
        __threadfence();
    }
    __syncthreads();
}

struct Ring {
    uint4 w[RING_UNITS][2];    // rows g and g + 8 of a 16x128 block (this thread's 32 nibbles of each)
    uint32_t s[RING_UNITS];    // their two bf16 scales
};

// Shared-memory carve-up of the matrix phases (the attention phase reuses the same bytes for its teams).
struct StackSmem {
    uint4 *fragments;    // [groups][4 words][staged lanes][4] activations in B-fragment order
    uint16_t *rows;      // [staged lanes][hidden] normalised rows before they are permuted
    float *correction;   // [groups][8] 136 * sum(x) per lane
    float *reduce;       // [2][warps][32 rows][8]
    float *partial;      // [32]
};

// ------------------------------------------------------------------------------------------ activation staging

// 16 consecutive chunks (uint4 = 8 bf16) are one (lane, group); chunk -> fragment slot of thread (g = lane, j)
// for word w is ((group * 4 + w) * staged + lane) * 4 + j, holding (v0,v4) (v1,v5) (v2,v6) (v3,v7): the B operands
// of the two MMAs that consume nibble pairs (0,4) (1,5) and (2,6) (3,7) of the matching weight word.
__device__ __forceinline__ void stage_chunk(const StackSmem &sm, uint4 raw, bool active, int chunk, int groups, int staged) {
    const int m = chunk / (groups * 16), rem = chunk - m * groups * 16, group = rem >> 4, part = rem & 15, j = part >> 2,
              word = part & 3;
    float sum = 0.0f;
    if (active) {
        uint4 out;
        out.x = __byte_perm(raw.x, raw.z, 0x5410);
        out.y = __byte_perm(raw.x, raw.z, 0x7632);
        out.z = __byte_perm(raw.y, raw.w, 0x5410);
        out.w = __byte_perm(raw.y, raw.w, 0x7632);
        sm.fragments[((group * 4 + word) * staged + m) * 4 + j] = out;
        sum = bf16_lo(raw.x) + bf16_hi(raw.x) + bf16_lo(raw.y) + bf16_hi(raw.y) + bf16_lo(raw.z) + bf16_hi(raw.z) + bf16_lo(raw.w) +
              bf16_hi(raw.w);
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    sum += __shfl_xor_sync(0xffffffffu, sum, 4);
    sum += __shfl_xor_sync(0xffffffffu, sum, 8);
    if (active && part == 0) sm.correction[group * 8 + m] = 136.0f * sum;
}

__device__ __forceinline__ void clear_unused_corrections(const StackSmem &sm, int groups, int staged) {
    for (int c = threadIdx.x; c < groups * 8; c += STACK_THREADS)
        if ((c & 7) >= staged) sm.correction[c] = 0.0f;
}

// Rows written by other CTAs of this launch ([lanes][width] bf16 in global memory, read through L2).
__device__ __forceinline__ void stage_global_rows(const StackSmem &sm, const uint16_t *x, int width, int staged) {
    const int groups = width >> 7, chunks = staged * groups * 16;
    for (int base = 0; base < chunks; base += STACK_THREADS) {
        const int chunk = base + threadIdx.x;
        const bool active = chunk < chunks;
        uint4 raw = make_uint4(0, 0, 0, 0);
        if (active) raw = __ldcg(reinterpret_cast<const uint4 *>(x) + chunk);  // chunk order == row-major order
        stage_chunk(sm, raw, active, active ? chunk : 0, groups, staged);
    }
    clear_unused_corrections(sm, groups, staged);
    __syncthreads();
}

// rms_norm_bf16.comp.template:49-72 of every staged lane (each CTA repeats it: 8 KB per lane from L2), then the
// normalised bf16 rows are permuted into fragment order.
__device__ __forceinline__ void stage_normalised_rows(const StackSmem &sm, const uint16_t *x, const uint16_t *weight, int width,
                                                      int staged, float eps, float offset) {
    const int words = width >> 1, warp = threadIdx.x >> 5;
    const uint32_t *weight_words = reinterpret_cast<const uint32_t *>(weight);
    uint32_t *row_words = reinterpret_cast<uint32_t *>(sm.rows);
    for (int m = 0; m < staged; m++) {
        const uint32_t *row = reinterpret_cast<const uint32_t *>(x) + static_cast<size_t>(m) * words;
        float sum = 0.0f;
        for (int word = threadIdx.x; word < words; word += STACK_THREADS) {
            uint32_t packed = __ldcg(row + word);
            float lo = bf16_lo(packed), hi = bf16_hi(packed);
            sum = fmaf(lo, lo, sum);
            sum = fmaf(hi, hi, sum);
        }
        sum = warp_sum(sum);
        __syncthreads();  // sm.partial of the previous lane has been read
        if ((threadIdx.x & 31) == 0) sm.partial[warp] = sum;
        __syncthreads();
        float total = 0.0f;
        for (int w = 0; w < STACK_WARPS; w++) total += sm.partial[w];
        const float inv_rms = 1.0f / sqrtf(total * (1.0f / static_cast<float>(width)) + eps);
        for (int word = threadIdx.x; word < words; word += STACK_THREADS) {
            uint32_t packed = __ldcg(row + word), w = __ldg(weight_words + word);
            float lo = bf16_lo(packed) * inv_rms * (bf16_lo(w) + offset);
            float hi = bf16_hi(packed) * inv_rms * (bf16_hi(w) + offset);
            row_words[static_cast<size_t>(m) * words + word] = pack_bf16(lo, hi);
        }
    }
    __syncthreads();
    const int groups = width >> 7, chunks = staged * groups * 16;
    for (int base = 0; base < chunks; base += STACK_THREADS) {
        const int chunk = base + threadIdx.x;
        const bool active = chunk < chunks;
        uint4 raw = make_uint4(0, 0, 0, 0);
        if (active) raw = reinterpret_cast<const uint4 *>(sm.rows)[chunk];
        stage_chunk(sm, raw, active, active ? chunk : 0, groups, staged);
    }
    clear_unused_corrections(sm, groups, staged);
    __syncthreads();
}

// ------------------------------------------------------------------------------------------ weight ring

template <int RT>
__device__ __forceinline__ void issue_item(Ring &ring, int first_unit, const TiledInt4 &matrix, int tile, int group) {
    const int lane = threadIdx.x & 31;
    const size_t block = (static_cast<size_t>(tile) * matrix.groups + group) * RT;
#pragma unroll
    for (int rt = 0; rt < RT; rt++) {
        const uint4 *src = matrix.weights + (block + rt) * 64 + lane;
        ring.w[first_unit + rt][0] = __ldg(src);
        ring.w[first_unit + rt][1] = __ldg(src + 32);
        ring.s[first_unit + rt] = __ldg(matrix.scales + (block + rt) * 8 + (lane >> 2));
    }
}

// A warp's items of one matrix: for each of the CTA's tiles (blockIdx.x, += gridDim.x) its groups (warp, += 16).
struct WarpItems {
    int per_tile, tiles, total;
};
__device__ __forceinline__ WarpItems warp_items(const TiledInt4 &matrix) {
    const int warp = threadIdx.x >> 5;
    WarpItems items;
    items.per_tile = matrix.groups > warp ? (matrix.groups - warp + STACK_WARPS - 1) / STACK_WARPS : 0;
    items.tiles = matrix.tiles > static_cast<int>(blockIdx.x) ? (matrix.tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x) : 0;
    items.total = items.per_tile * items.tiles;
    return items;
}
__device__ __forceinline__ void issue_numbered(Ring &ring, int first_unit, const TiledInt4 &matrix, const WarpItems &items, int number,
                                               int rt_count) {
    int tile_index = 0;
    while (number >= items.per_tile) {
        number -= items.per_tile;
        tile_index++;
    }
    const int tile = blockIdx.x + tile_index * gridDim.x, group = (threadIdx.x >> 5) + number * STACK_WARPS;
    if (rt_count == 2) issue_item<2>(ring, first_unit, matrix, tile, group);
    else issue_item<1>(ring, first_unit, matrix, tile, group);
}

// Before a matrix phase: whatever of the warp's first RING_UNITS / RT items the previous phase did not already
// request (bit i of `mask`) is requested now, ahead of the activation staging.
template <int RT>
__device__ __forceinline__ void prefetch_entry(Ring &ring, uint32_t &mask, const TiledInt4 &matrix) {
    constexpr int SLOTS = RING_UNITS / RT;
    const WarpItems items = warp_items(matrix);
#pragma unroll
    for (int slot = 0; slot < SLOTS; slot++)
        if (!((mask >> slot) & 1u) && slot < items.total) issue_numbered(ring, slot * RT, matrix, items, slot, RT);
    mask = 0;
}

// ------------------------------------------------------------------------------------------ matrix phase

// Streams the CTA's tiles of `current` (its first RING_UNITS / RT items per warp already requested).  While the
// last items are consumed the freed ring units are refilled with the first items of `next` (NRT = its rt count,
// 0 = none); `mask` returns which of them were requested.  epilogue(tile, r, m, sums) gets, for lane m, the
// results of MMA rows r and r + 8 of the tile (sums[rt][0], sums[rt][1]) and is run by 64 threads.
template <int RT, int NRT, class Epilogue>
__device__ __forceinline__ void matrix_phase(const TiledInt4 current, const TiledInt4 next, Ring &ring, uint32_t &mask,
                                             const StackSmem &sm, int staged, int lanes, int &parity, Epilogue epilogue) {
    constexpr int SLOTS = RING_UNITS / RT;
    constexpr int NSLOTS = NRT > 0 ? RING_UNITS / NRT : 0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, j = lane & 3;
    const WarpItems items = warp_items(current);
    WarpItems next_items = items;
    if (NRT > 0) next_items = warp_items(next);
    const int tiles_of_cta = items.tiles;

    int issued = items.total < SLOTS ? items.total : SLOTS;
    int issue_gi = issued, issue_tile = blockIdx.x;
    while (items.per_tile > 0 && issue_gi >= items.per_tile) {
        issue_gi -= items.per_tile;
        issue_tile += gridDim.x;
    }
    uint32_t freed = 0, requested = 0;

    const int ge = g < staged ? g : 0;  // lanes beyond the batch recompute lane 0; their results are dropped
    const uint4 *xlane = sm.fragments + ge * 4 + j;
    float acc[RT][4];
#pragma unroll
    for (int rt = 0; rt < RT; rt++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[rt][i] = 0.0f;
    int cur_tile = blockIdx.x, cur_gi = 0;

    auto finish_tile = [&]() {
        float *mine = sm.reduce + static_cast<size_t>((parity * STACK_WARPS + warp) * 32) * 8;
#pragma unroll
        for (int rt = 0; rt < RT; rt++) {
            *reinterpret_cast<float2 *>(mine + (rt * 16 + g) * 8 + 2 * j) = make_float2(acc[rt][0], acc[rt][1]);
            *reinterpret_cast<float2 *>(mine + (rt * 16 + g + 8) * 8 + 2 * j) = make_float2(acc[rt][2], acc[rt][3]);
            acc[rt][0] = acc[rt][1] = acc[rt][2] = acc[rt][3] = 0.0f;
        }
        __syncthreads();
        if (threadIdx.x < 64) {
            const int r = threadIdx.x >> 3, m = threadIdx.x & 7;
            if (m < lanes) {
                const float *src = sm.reduce + static_cast<size_t>(parity * STACK_WARPS * 32 + r) * 8 + m;
                float sums[RT][2];
#pragma unroll
                for (int rt = 0; rt < RT; rt++) sums[rt][0] = sums[rt][1] = 0.0f;
#pragma unroll
                for (int w = 0; w < STACK_WARPS; w++)
#pragma unroll
                    for (int rt = 0; rt < RT; rt++) {
                        sums[rt][0] += src[(w * 32 + rt * 16) * 8];
                        sums[rt][1] += src[(w * 32 + rt * 16 + 8) * 8];
                    }
                epilogue(cur_tile, r, m, sums);
            }
        }
        parity ^= 1;
        cur_gi = 0;
        cur_tile += gridDim.x;
    };

    if (items.per_tile == 0) {
        // a warp without groups of this K still takes part in every tile's reduction
        for (int t = 0; t < tiles_of_cta; t++) finish_tile();
    }
    for (int it = 0; it < items.total;) {
#pragma unroll
        for (int slot = 0; slot < SLOTS; slot++) {
            if (it >= items.total) break;
            const int group = warp + cur_gi * STACK_WARPS;
            uint4 b[4];
#pragma unroll
            for (int word = 0; word < 4; word++) b[word] = xlane[(group * 4 + word) * staged * 4];
            const float2 bias = *reinterpret_cast<const float2 *>(sm.correction + group * 8 + 2 * j);
#pragma unroll
            for (int rt = 0; rt < RT; rt++) {
                const int unit = slot * RT + rt;
                float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                const uint32_t wa[4] = {ring.w[unit][0].x, ring.w[unit][0].y, ring.w[unit][0].z, ring.w[unit][0].w};
                const uint32_t wb[4] = {ring.w[unit][1].x, ring.w[unit][1].y, ring.w[unit][1].z, ring.w[unit][1].w};
#pragma unroll
                for (int word = 0; word < 4; word++) {
                    mma_bf16_16816(c, biased_pair(wa[word], 0), biased_pair(wb[word], 0), biased_pair(wa[word], 4),
                                   biased_pair(wb[word], 4), b[word].x, b[word].y);
                    mma_bf16_16816(c, biased_pair(wa[word], 8), biased_pair(wb[word], 8), biased_pair(wa[word], 12),
                                   biased_pair(wb[word], 12), b[word].z, b[word].w);
                }
                const float sa = __uint_as_float(ring.s[unit] << 16), sb = __uint_as_float(ring.s[unit] & 0xffff0000u);
                acc[rt][0] = fmaf(sa, c[0] - bias.x, acc[rt][0]);
                acc[rt][1] = fmaf(sa, c[1] - bias.y, acc[rt][1]);
                acc[rt][2] = fmaf(sb, c[2] - bias.x, acc[rt][2]);
                acc[rt][3] = fmaf(sb, c[3] - bias.y, acc[rt][3]);
            }
            if (issued < items.total) {
                issue_item<RT>(ring, slot * RT, current, issue_tile, warp + issue_gi * STACK_WARPS);
                issued++;
                if (++issue_gi == items.per_tile) {
                    issue_gi = 0;
                    issue_tile += gridDim.x;
                }
            } else if (NRT > 0) {
                freed |= ((1u << RT) - 1u) << (slot * RT);
#pragma unroll
                for (int ns = 0; ns < NSLOTS; ns++) {
                    const uint32_t need = ((1u << NRT) - 1u) << (ns * NRT);
                    if (!((requested >> ns) & 1u) && (freed & need) == need && ns < next_items.total) {
                        issue_numbered(ring, ns * NRT, next, next_items, ns, NRT);
                        requested |= 1u << ns;
                    }
                }
            }
            it++;
            if (++cur_gi == items.per_tile) finish_tile();
        }
    }
    mask = NRT > 0 ? requested : 0u;
}

// ------------------------------------------------------------------------------------------ epilogues

// q/k/v: tiles [0, q_tiles) are q, the next k_tiles are k, the rest v.  q and k rows arrive as rotary partners
// (rotary_bf16.comp.template:99-109, non-interleaved, rotary width = head width: five bf16 roundings); k and v
// are written into the lane's KV page (append_gqa_attention_bf16.comp.template:189-215), q into the q buffer.
struct QkvEpilogue {
    int q_tiles, k_tiles, head_width, q_heads;
    uint16_t *q;
    KvLayer kv;
    LaneTable lanes_meta;
    const uint32_t *rope_table;
    uint32_t rope_positions;

    __device__ __forceinline__ void operator()(int tile, int r, int m, const float (&sums)[1][2]) const {
        const float low = round_bf16(sums[0][0]), high = round_bf16(sums[0][1]);
        const uint32_t position = lanes_meta.position[m];
        const int slot = lanes_meta.slot[m];
        if (tile < q_tiles + k_tiles) {
            const bool is_q = tile < q_tiles;
            const int local = is_q ? tile : tile - q_tiles;
            const int tiles_per_head = head_width >> 4, half = head_width >> 1;
            const int head = local / tiles_per_head, d = 8 * (local % tiles_per_head) + r;
            const uint32_t packed = __ldg(rope_table + static_cast<size_t>(position % rope_positions) * half + d);
            const float cosine = bf16_lo(packed), sine = bf16_hi(packed);
            const uint16_t out_low = static_cast<uint16_t>(f32_to_bf16_bits(round_bf16(low * cosine) + round_bf16(-high * sine)));
            const uint16_t out_high = static_cast<uint16_t>(f32_to_bf16_bits(round_bf16(high * cosine) + round_bf16(low * sine)));
            if (is_q) {
                uint16_t *dst = q + (static_cast<size_t>(m) * q_heads + head) * head_width + d;
                dst[0] = out_low;
                dst[half] = out_high;
            } else if (slot >= 0 && kv.capacity != 0) {
                uint16_t *dst = kv.pool + kv_token_offset(kv, slot, position % kv.capacity, head, false) + d;
                dst[0] = out_low;
                dst[half] = out_high;
            }
        } else if (slot >= 0 && kv.capacity != 0) {
            const int row = (tile - q_tiles - k_tiles) * 16 + r;
            const int head = row / head_width, d = row % head_width;
            uint16_t *dst = kv.pool + kv_token_offset(kv, slot, position % kv.capacity, head, true) + d;
            dst[0] = static_cast<uint16_t>(f32_to_bf16_bits(sums[0][0]));
            dst[8] = static_cast<uint16_t>(f32_to_bf16_bits(sums[0][1]));
        }
    }
};

// linear + residual_add (add_bf16.comp.template:17-24): bf16(bf16(product) + residual), in place.
struct ResidualEpilogue {
    uint16_t *hidden;
    int width;
    __device__ __forceinline__ void operator()(int tile, int r, int m, const float (&sums)[1][2]) const {
        uint16_t *dst = hidden + static_cast<size_t>(m) * width + tile * 16 + r;
        const float first = bf16_bits_to_f32(__ldcg(dst)), second = bf16_bits_to_f32(__ldcg(dst + 8));
        dst[0] = static_cast<uint16_t>(f32_to_bf16_bits(round_bf16(sums[0][0]) + first));
        dst[8] = static_cast<uint16_t>(f32_to_bf16_bits(round_bf16(sums[0][1]) + second));
    }
};

// gate/up pair: bf16(silu_bf16(bf16 gate) * bf16 up) (silu_multiply_bf16.comp.template:30-52).
struct SiluEpilogue {
    uint16_t *activation;
    int width;
    __device__ __forceinline__ void operator()(int tile, int r, int m, const float (&sums)[2][2]) const {
        uint16_t *dst = activation + static_cast<size_t>(m) * width + tile * 16 + r;
        dst[0] = static_cast<uint16_t>(f32_to_bf16_bits(rounded_silu(round_bf16(sums[0][0])) * round_bf16(sums[1][0])));
        dst[8] = static_cast<uint16_t>(f32_to_bf16_bits(rounded_silu(round_bf16(sums[0][1])) * round_bf16(sums[1][1])));
    }
};

// ------------------------------------------------------------------------------------------ the kernel

struct StackArgs {
    const StackLayer *layers;
    int layer_count;
    StackShape shape;
    StackBuffers buffers;
    LaneTable lanes_meta;
    int lanes, lanes_per_stream, split_tokens, max_splits;
};

struct StackSmemLayout {
    size_t fragments, rows, correction, reduce, partial, total;
};
__host__ __device__ inline StackSmemLayout stack_smem_layout(const StackShape &shape, int staged, size_t attention_bytes) {
    const size_t q_width = static_cast<size_t>(shape.q_heads) * shape.head_width;
    size_t widest = shape.hidden > shape.ffn ? shape.hidden : shape.ffn;
    if (q_width > widest) widest = q_width;
    size_t region = static_cast<size_t>(staged) * widest * 2;
    const size_t norm_region = static_cast<size_t>(staged) * shape.hidden * 2 * 2;  // fragments + plain rows
    if (norm_region > region) region = norm_region;
    StackSmemLayout layout;
    layout.fragments = 0;
    layout.rows = static_cast<size_t>(staged) * shape.hidden * 2;
    layout.correction = region;
    layout.reduce = layout.correction + (widest >> 7) * 8 * sizeof(float);
    layout.partial = layout.reduce + static_cast<size_t>(2) * STACK_WARPS * 32 * 8 * sizeof(float);
    layout.total = layout.partial + 32 * sizeof(float);
    if (attention_bytes > layout.total) layout.total = attention_bytes;
    return layout;
}

template <int GROUP>
struct AttentionTeam {
    static constexpr int QL = GROUP >= 8 ? 2 : ATTENTION_QL;
};

template <int HD, int GROUP>
__global__ void __launch_bounds__(STACK_THREADS, 1) decode_stack_kernel(const StackArgs a) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    constexpr int QL = AttentionTeam<GROUP>::QL;
    const StackShape &shape = a.shape;
    const int lanes = a.lanes, staged = lanes < 8 ? lanes : 8;
    const StackSmemLayout layout = stack_smem_layout(shape, staged, 0);
    StackSmem sm;
    sm.fragments = reinterpret_cast<uint4 *>(smem_raw + layout.fragments);
    sm.rows = reinterpret_cast<uint16_t *>(smem_raw + layout.rows);
    sm.correction = reinterpret_cast<float *>(smem_raw + layout.correction);
    sm.reduce = reinterpret_cast<float *>(smem_raw + layout.reduce);
    sm.partial = reinterpret_cast<float *>(smem_raw + layout.partial);

    const int q_width = shape.q_heads * HD;
    unsigned int target = 0;
    unsigned int *counter = a.buffers.barrier;
    int *error_flag = a.buffers.error_flag;
    int parity = 0;
    uint32_t mask = 0;
    Ring ring;

    auto stamp = [&](int layer, int phase) {
        if (a.buffers.timing != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            a.buffers.timing[layer * 8 + phase] = now;
        }
    };
    for (int layer = 0; layer < a.layer_count; layer++) {
        const StackLayer *spec = a.layers + layer;
        stamp(layer, 0);
        const TiledInt4 qkv = spec->qkv, o = spec->o, gate_up = spec->gate_up, down = spec->down;
        const KvLayer kv = spec->kv;

        // ---- rms_norm + q/k/v + RoPE + KV append
        prefetch_entry<1>(ring, mask, qkv);
        stage_normalised_rows(sm, a.buffers.hidden, spec->input_norm, shape.hidden, staged, shape.eps, shape.norm_offset);
        {
            QkvEpilogue epilogue;
            epilogue.q_tiles = q_width >> 4;
            epilogue.k_tiles = (shape.kv_heads * HD) >> 4;
            epilogue.head_width = HD;
            epilogue.q_heads = shape.q_heads;
            epilogue.q = a.buffers.q;
            epilogue.kv = kv;
            epilogue.lanes_meta = a.lanes_meta;
            epilogue.rope_table = shape.rope_table;
            epilogue.rope_positions = shape.rope_positions;
            matrix_phase<1, 0>(qkv, qkv, ring, mask, sm, staged, lanes, parity, epilogue);
        }
        grid_barrier(counter, target, error_flag);
        stamp(layer, 1);

        // ---- attention: (kv head, split, stream x lane group) items over all teams of the grid
        {
            const int team = threadIdx.x >> 7, team_tid = threadIdx.x & 127;
            const int streams = lanes / a.lanes_per_stream;
            const int group_slots = streams * ((a.lanes_per_stream + QL - 1) / QL);
            const int total = shape.kv_heads * a.max_splits * group_slots;
            uint8_t *team_smem = smem_raw + static_cast<size_t>(team) * attention_team_smem<HD, GROUP, QL>();
            for (int item = blockIdx.x * ATTENTION_TEAMS + team; item < total; item += gridDim.x * ATTENTION_TEAMS) {
                const int kv_head = item % shape.kv_heads, rest = item / shape.kv_heads;
                const int split = rest % a.max_splits, group_slot = rest / a.max_splits;
                attention_tile_body<HD, GROUP, QL, true>(a.buffers.q, kv, a.lanes_meta, lanes, a.lanes_per_stream, shape.q_heads,
                                                         shape.attention_scale, a.split_tokens, a.max_splits,
                                                         a.buffers.attention_scratch, kv_head, split, group_slot, team_smem, team_tid,
                                                         1 + team);
            }
        }
        prefetch_entry<1>(ring, mask, o);
        grid_barrier(counter, target, error_flag);
        stamp(layer, 2);
        {
            const int pairs = lanes * shape.q_heads;
            for (int pair = blockIdx.x * STACK_WARPS + (threadIdx.x >> 5); pair < pairs; pair += gridDim.x * STACK_WARPS)
                attention_merge_pair<true>(a.buffers.attention_scratch, a.buffers.attention_out, kv, a.lanes_meta, pair, threadIdx.x & 31,
                                           shape.q_heads, HD, a.split_tokens, a.max_splits);
        }
        grid_barrier(counter, target, error_flag);
        stamp(layer, 3);

        // ---- o projection + residual
        stage_global_rows(sm, a.buffers.attention_out, q_width, staged);
        matrix_phase<1, 2>(o, gate_up, ring, mask, sm, staged, lanes, parity, ResidualEpilogue{a.buffers.hidden, shape.hidden});
        grid_barrier(counter, target, error_flag);
        stamp(layer, 4);

        // ---- rms_norm + gate/up + SiLU multiply
        prefetch_entry<2>(ring, mask, gate_up);
        stage_normalised_rows(sm, a.buffers.hidden, spec->post_norm, shape.hidden, staged, shape.eps, shape.norm_offset);
        matrix_phase<2, 1>(gate_up, down, ring, mask, sm, staged, lanes, parity, SiluEpilogue{a.buffers.activation, shape.ffn});
        grid_barrier(counter, target, error_flag);
        stamp(layer, 5);

        // ---- down projection + residual
        prefetch_entry<1>(ring, mask, down);
        stage_global_rows(sm, a.buffers.activation, shape.ffn, staged);
        if (layer + 1 < a.layer_count) {
            const TiledInt4 following = a.layers[layer + 1].qkv;
            matrix_phase<1, 1>(down, following, ring, mask, sm, staged, lanes, parity, ResidualEpilogue{a.buffers.hidden, shape.hidden});
        } else {
            matrix_phase<1, 0>(down, down, ring, mask, sm, staged, lanes, parity, ResidualEpilogue{a.buffers.hidden, shape.hidden});
        }
        grid_barrier(counter, target, error_flag);
        stamp(layer, 6);
    }

    // The last CTA to leave rearms the barrier words for the next launch (every CTA has passed its last barrier
    // before it counts itself out).
    if (threadIdx.x == 0) {
        const unsigned int gone = atomicAdd(counter + 1, 1u);
        if (gone == gridDim.x - 1) {
            counter[0] = 0u;
            counter[1] = 0u;
            __threadfence();
        }
    }
}

template <int HD, int GROUP>
cudaError_t launch_instance(const StackArgs &args, size_t smem, cudaStream_t stream) {
    static int configured_device = -1, sm_count = 0;
    int device = 0;
    cudaError_t status = cudaGetDevice(&device);
    if (status != cudaSuccess) return status;
    if (configured_device != device) {
        status = cudaFuncSetAttribute(decode_stack_kernel<HD, GROUP>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (status != cudaSuccess) return status;
        status = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
        if (status != cudaSuccess) return status;
        configured_device = device;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(sm_count);
    config.blockDim = dim3(STACK_THREADS);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeCooperative;  // all CTAs co-resident: they wait on one another
    attribute[0].val.cooperative = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, decode_stack_kernel<HD, GROUP>, args);
}

template <int HD, int GROUP>
size_t attention_bytes_of() {
    return ATTENTION_TEAMS * attention_team_smem<HD, GROUP, AttentionTeam<GROUP>::QL>();
}

bool instance_smem(const StackShape &shape, int lanes, size_t *bytes) {
    const int group = shape.kv_heads > 0 ? shape.q_heads / shape.kv_heads : 0;
    size_t attention = 0;
    if (shape.head_width == 128 && group == 4) attention = attention_bytes_of<128, 4>();
    else if (shape.head_width == 128 && group == 8) attention = attention_bytes_of<128, 8>();
    else if (shape.head_width == 64 && group == 4) attention = attention_bytes_of<64, 4>();
    else if (shape.head_width == 32 && group == 2) attention = attention_bytes_of<32, 2>();
    else return false;
    *bytes = stack_smem_layout(shape, lanes < 8 ? lanes : 8, attention).total;
    return true;
}

}  // namespace

cudaError_t launch_int4_tile_major(const RelayoutSegment *segments, int count, bool pair, int k, uint4 *weights_out,
                                   uint32_t *scales_out, cudaStream_t stream) {
    if (count < 1 || count > 3 || (pair && count != 2) || k % 128 != 0) return cudaErrorInvalidValue;
    RelayoutArgs args = {};
    args.count = count;
    args.pair = pair ? 1 : 0;
    args.k = k;
    int tiles = 0;
    for (int i = 0; i < count; i++) {
        if (segments[i].rows % 16 != 0) return cudaErrorInvalidValue;
        if (segments[i].rope_head_width > 0 && (segments[i].rope_head_width % 16 != 0 || segments[i].rows % segments[i].rope_head_width != 0))
            return cudaErrorInvalidValue;
        args.segment[i] = segments[i];
        args.first_tile[i] = tiles;
        if (!pair || i == 0) tiles += segments[i].rows / 16;
    }
    if (pair && segments[0].rows != segments[1].rows) return cudaErrorInvalidValue;
    args.first_tile[count] = tiles;
    args.tiles = tiles;
    int4_tile_major_kernel<<<148 * 4, 256, 0, stream>>>(args, weights_out, scales_out);
    return cudaGetLastError();
}

bool decode_stack_supported(const StackShape &shape, int lanes, size_t *smem_bytes) {
    size_t bytes = 0;
    if (lanes < 1 || lanes > 8) return false;
    if (shape.hidden % 128 != 0 || shape.ffn % 128 != 0 || (shape.q_heads * shape.head_width) % 128 != 0) return false;
    if (!instance_smem(shape, lanes, &bytes)) return false;
    if (bytes > 227 * 1024) return false;
    if (smem_bytes) *smem_bytes = bytes;
    return true;
}

cudaError_t launch_decode_stack(const StackLayer *layers_device, int layer_count, const StackShape &shape,
                                const StackBuffers &buffers, const LaneTable &lanes_meta, int lanes, int lanes_per_stream,
                                int split_tokens, int max_splits, cudaStream_t stream) {
    size_t smem = 0;
    if (!decode_stack_supported(shape, lanes, &smem) || lanes_per_stream <= 0 || lanes % lanes_per_stream != 0 || layer_count < 1)
        return cudaErrorInvalidValue;
    StackArgs args;
    args.layers = layers_device;
    args.layer_count = layer_count;
    args.shape = shape;
    args.buffers = buffers;
    args.lanes_meta = lanes_meta;
    args.lanes = lanes;
    args.lanes_per_stream = lanes_per_stream;
    args.split_tokens = split_tokens;
    args.max_splits = max_splits;
    const int group = shape.q_heads / shape.kv_heads;
    if (shape.head_width == 128 && group == 4) return launch_instance<128, 4>(args, smem, stream);
    if (shape.head_width == 128 && group == 8) return launch_instance<128, 8>(args, smem, stream);
    if (shape.head_width == 64 && group == 4) return launch_instance<64, 4>(args, smem, stream);
    return launch_instance<32, 2>(args, smem, stream);
}

}  // namespace nerve

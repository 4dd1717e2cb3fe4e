// Persistent decode stack: one cooperative launch runs every layer of a dense INT4 g128 Llama-style stack
// (rms_norm, q/k/v, RoPE, KV append, attention, o + residual, rms_norm, gate/up + SiLU, down + residual:
// the kernel list of one reference layer component, runtime-rs/shaders/*.comp.template) for a batch of at most
// 8 lanes - the verify batch and the draft / single-tick steps of the speculative decode cycle.
//
// Why one launch: at these batch sizes a layer is ~112 MB of weights (~17 us of HBM time) cut into a dozen
// dependent steps; as separate kernels every step pays a launch, a pipeline fill and a drain (~6 us each,
// measured), which is several times the streaming time.  Here one CTA per SM stays resident, keeps a ring of
// asynchronous copies of packed weights in flight across step boundaries (weights do not depend on activations,
// so the next matrix is already streaming while the grid waits at a barrier), and the steps are separated by
// grid-wide barriers (bounded spins on one global counter).
//
// Data layout:
//  * weights: a tile-major copy made at mount - [tile of 16 rows][group of 128 columns][rt][half][lane] uint4,
//    i.e. exactly the order in which a warp's two 16-byte loads consume them (each load is 512 contiguous
//    bytes; a tile is K/128 contiguous KB).  q and k tiles pair row d with row d + head_width/2, so RoPE runs in
//    the q/k/v epilogue and K, V go straight into the KV pages.
//  * activations of a step: staged once per CTA in shared memory in mma.sync B-fragment order, together with
//    -24 * sum(x) per (lane, group): the nibbles are fed to the tensor cores as bf16 16+q (one shift and one lop3
//    per pair, no subtract) and the bias 16+8 is taken out per group by starting the accumulation from that sum.
//  * a matrix tile is computed by all 16 warps of a CTA (each takes every 16th group of K), reduced through
//    shared memory, and finished by 128 epilogue threads (one per row and lane).
//  * attention: a team of four warps per (kv head, 64-token split, lane group) on the tensor cores, partials
//    merged per (lane, head) by one warp after a barrier.
//  * tensor parallelism (the EXCHANGE instances): o and down leave f32 partial sums in the rank's exchange buffer;
//    the ranks meet at a two-level barrier over NVLink and add each other's partials up from peer memory.
// The per-layer code is one loop over the four matrix steps with run-time matrix / epilogue selection: the
// straight-line form of the same steps did not fit the instruction cache and spent most of its time refetching.
#include <cstdlib>

#include "attention_body.cuh"
#include "common.cuh"
#include "kernels.cuh"

namespace nerve {

namespace {

constexpr int STACK_WARPS = 16;
constexpr int STACK_THREADS = STACK_WARPS * 32;
constexpr int MAX_RING_UNITS = 8;      // 16x128 weight blocks (1 KB + scales) a warp keeps in flight, at most
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

// The same with a zero accumulator coming in (starts a chain without clearing registers first).
__device__ __forceinline__ void mma_bf16_16816_first(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                                     uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

// Nibble pair k of `word` (bits 4k..4k+3 and 16+4k..16+4k+3) -> bf16x2 (16 + q, 16 + q'): with the nibble in
// mantissa bits 3..6 under exponent 2^4, 0x4180 | q << 3 is exactly 16 + q.  One shift and one lop3 per pair; the
// offset 16 (+ 8 of the symmetric INT4 code) leaves the accumulator as 24 * sum(x) per group, taken out afterwards.
template <int PAIR>
__device__ __forceinline__ uint32_t biased_pair(uint32_t word) {
    uint32_t out;
    const uint32_t aligned = PAIR == 0 ? word << 3 : word >> (4 * PAIR - 3);
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(out) : "r"(aligned), "n"(0x00780078), "n"(0x41804180));
    return out;
}
constexpr float NIBBLE_BIAS = 24.0f;

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
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");  // covers the CTA's writes before the barrier above
        unsigned int spins = 0;
        while (load_acquire(counter) < target) {
            if (++spins > BARRIER_SPIN_LIMIT) {
                atomicExch(error_flag, 2);
                break;
            }
            if ((spins & 63u) == 0 && *reinterpret_cast<volatile int *>(error_flag) != 0) break;
        }
    }
    __syncthreads();
}

// All CTAs of all tensor-parallel ranks meet here, in two levels: the CTAs of this GPU count themselves in on a
// local word; the last one to arrive tells every peer (one system-scope store of the exchange number per peer, over
// NVLink); every CTA then waits until all local CTAs and every peer have done so.  One remote write per peer and
// exchange: arrivals of 148 CTAs on one remote word would queue up on the link.  `exchange_number` counts the
// exchanges of this and all earlier launches; all words only grow.  What the CTAs wrote into their rank's exchange
// buffer before the call is visible to the peers after it.  Every wait is bounded; a rank that never shows up ends
// the launch with the error flag set.
// Control words of a rank (unsigned long long, behind its exchange buffer): [0] local arrivals, [1] unused,
// [2] exchanges consumed by earlier launches, [8 + s] the exchange number rank s has reached.
constexpr unsigned int EXCHANGE_SPIN_LIMIT = 1u << 24;  // about ten seconds of polling: ranks start their launches a host jitter apart
constexpr int TP_WORD_ARRIVALS = 0, TP_WORD_GO = 1, TP_WORD_CONSUMED = 2, TP_WORD_PEER = 8;

__device__ __forceinline__ unsigned long long load_acquire_sys(const unsigned long long *address) {
    unsigned long long value;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(value) : "l"(address) : "memory");
    return value;
}
__device__ __forceinline__ unsigned long long load_acquire_gpu(const unsigned long long *address) {
    unsigned long long value;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(value) : "l"(address) : "memory");
    return value;
}

__device__ __noinline__ void exchange_barrier(const StackTp &tp, unsigned long long &exchange_number, int *error_flag) {
    __syncthreads();
    if (threadIdx.x == 0) {
        exchange_number += 1;
        unsigned long long *mine = tp.counter[tp.rank];
        // release: the CTA's writes before the barrier above; acquire: the last to arrive takes over everybody's
        unsigned long long before;
        asm volatile("atom.acq_rel.gpu.global.add.u64 %0, [%1], 1;" : "=l"(before) : "l"(mine + TP_WORD_ARRIVALS) : "memory");
        unsigned int spins = 0;
        bool gave_up = false;
        if (before + 1 == exchange_number * gridDim.x) {
            // the last CTA of this GPU: everything this rank wrote for the exchange is in memory; the system-scope
            // release stores publish it to the peers
            for (int r = 0; r < tp.size; r++)
                if (r != tp.rank)
                    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(tp.counter[r] + TP_WORD_PEER + tp.rank), "l"(exchange_number) : "memory");
        }
        // every CTA waits for the same two things itself (no hop through a go word): all CTAs of this GPU have
        // arrived, and every peer has said so of its own
        const unsigned long long all_here = exchange_number * gridDim.x;
        while (!gave_up && load_acquire_gpu(mine + TP_WORD_ARRIVALS) < all_here) {
            if (++spins > EXCHANGE_SPIN_LIMIT) {
                atomicExch(error_flag, 2);
                gave_up = true;
            } else if ((spins & 63u) == 0 && *reinterpret_cast<volatile int *>(error_flag) != 0) {
                gave_up = true;
            }
        }
        for (int r = 0; r < tp.size && !gave_up; r++) {
            if (r == tp.rank) continue;
            while (load_acquire_sys(mine + TP_WORD_PEER + r) < exchange_number) {
                if (++spins > EXCHANGE_SPIN_LIMIT) {
                    atomicExch(error_flag, 2);
                    gave_up = true;
                    break;
                }
                if ((spins & 63u) == 0 && *reinterpret_cast<volatile int *>(error_flag) != 0) {
                    gave_up = true;
                    break;
                }
            }
        }
    }
    __syncthreads();
}

// After an exchange: hidden = bf16(bf16(sum over ranks of the partial sums) + hidden) for this CTA's share of the
// [lanes][width] elements, four at a time (add_bf16.comp.template:17-24 on the all-reduced linear output).  Every
// rank keeps its own partial sums in its own buffer and the others read them from there (peer loads, all in flight
// at once: one NVLink round trip).  The partials are added in rank order on every rank, so the replicated residual
// streams stay bit-identical.
__device__ __noinline__ void reduce_exchanged(const StackTp &tp, int parity, uint16_t *hidden, int lanes, int width) {
    const int per_lane = width >> 2, items = lanes * per_lane;
    for (int item = blockIdx.x * STACK_THREADS + threadIdx.x; item < items; item += gridDim.x * STACK_THREADS) {
        const int m = item / per_lane, quad = item - m * per_lane;
        const size_t offset = (static_cast<size_t>(parity) * 8 + m) * per_lane + quad;
        float4 part[STACK_TP_MAX_RANKS];
#pragma unroll
        for (int r = 0; r < STACK_TP_MAX_RANKS; r++)
            if (r < tp.size) part[r] = __ldcg(reinterpret_cast<const float4 *>(tp.exchange[r]) + offset);
        uint2 *destination = reinterpret_cast<uint2 *>(hidden) + static_cast<size_t>(m) * per_lane + quad;
        const uint2 residual = __ldcg(destination);
        float4 sum = part[0];
#pragma unroll
        for (int r = 1; r < STACK_TP_MAX_RANKS; r++)
            if (r < tp.size) {
                sum.x += part[r].x;
                sum.y += part[r].y;
                sum.z += part[r].z;
                sum.w += part[r].w;
            }
        uint2 out;
        out.x = pack_bf16(round_bf16(sum.x) + bf16_lo(residual.x), round_bf16(sum.y) + bf16_hi(residual.x));
        out.y = pack_bf16(round_bf16(sum.z) + bf16_lo(residual.y), round_bf16(sum.w) + bf16_hi(residual.y));
        *destination = out;
    }
}

// Shared-memory carve-up of the matrix phases.
struct StackSmem {
    uint4 *fragments;    // [groups][4 words][staged lanes][4] activations in B-fragment order
    uint16_t *rows;      // [staged lanes][hidden] normalised rows before they are permuted
    float *correction;   // [groups][8] -24 * sum(x) per lane
    float *reduce;       // [2][warps][32 rows][8]
    float *partial;      // [8 lanes][warps]
    uint8_t *ring;       // [warps][RING_UNITS][RING_UNIT_BYTES] packed weights in flight (asynchronous copies)
};

// ------------------------------------------------------------------------------------------ weight stream
// Every thread copies its own 2 x 16 bytes of packed weights and its 4-byte scale pair of a 16x128 block with
// cp.async and later reads back exactly those bytes, so no thread waits on another: cp.async.wait_group is the
// only synchronisation.  Copy groups complete in issue order and blocks are consumed in issue order, also
// across matrices, so "all but the newest n groups" is always the right thing to wait for.  A warp's producer
// cursor runs ahead of its consumer by up to RING_UNITS blocks and crosses into the next matrix as soon as the
// current one is fully requested: the next phase's first weights are in flight while the grid is still at the
// barrier in front of it.

constexpr int RING_UNIT_BYTES = 2 * 512 + 128;

// cp.async with shared-space destination addresses and byte offsets folded into the instruction.
template <int DST_OFFSET, int SRC_OFFSET>
__device__ __forceinline__ void async_copy16(uint32_t shared_address, const void *source) {
    asm volatile("cp.async.cg.shared.global [%0+%2], [%1+%3], 16;" ::"r"(shared_address), "l"(source), "n"(DST_OFFSET), "n"(SRC_OFFSET) : "memory");
}
template <int SRC_OFFSET>
__device__ __forceinline__ void async_copy4(uint32_t shared_address, const void *source) {
    asm volatile("cp.async.ca.shared.global [%0], [%1+%2], 4;" ::"r"(shared_address), "l"(source), "n"(SRC_OFFSET) : "memory");
}
__device__ __forceinline__ void async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// Waits until at most `newer` of this thread's copy groups are still in flight.
__device__ __forceinline__ void async_wait(int newer) {
    switch (newer) {
    case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
    case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
    case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
    case 5: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
    case 6: asm volatile("cp.async.wait_group 6;" ::: "memory"); break;
    default: asm volatile("cp.async.wait_group 7;" ::: "memory"); break;
    }
}

// Waits for the oldest of this thread's `in_flight` (>= 1) copy groups; the usual depths are tested first.
__device__ __forceinline__ void async_wait_oldest(int in_flight) {
    if (in_flight == 4) asm volatile("cp.async.wait_group 3;" ::: "memory");
    else if (in_flight == 2) asm volatile("cp.async.wait_group 1;" ::: "memory");
    else async_wait(in_flight - 1);
}
// Shared-memory loads by shared-space address (32-bit address arithmetic, offsets folded into the instruction).
template <int OFFSET>
__device__ __forceinline__ uint4 shared_load16(uint32_t address) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(address), "n"(OFFSET) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t shared_load4(uint32_t address) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(address) : "memory");
    return v;
}
__device__ __forceinline__ float2 shared_load_float2(uint32_t address) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(address) : "memory");
    return v;
}

// One matrix as a warp sees it: for each of the CTA's tiles (blockIdx.x, += gridDim.x) the warp's groups
// (warp, += 16); an item is `rt` ring units (rt = 2 for a gate/up pair).
struct MatrixWalk {
    TiledInt4 matrix;
    int rt, per_tile, tiles, total;
};
__device__ __forceinline__ MatrixWalk walk_of(const TiledInt4 &matrix, int rt) {
    const int warp = threadIdx.x >> 5;
    MatrixWalk walk;
    walk.matrix = matrix;
    walk.rt = rt;
    walk.per_tile = matrix.groups > warp ? (matrix.groups - warp + STACK_WARPS - 1) / STACK_WARPS : 0;
    walk.tiles = matrix.tiles > static_cast<int>(blockIdx.x)
                     ? (matrix.tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x)
                     : 0;
    walk.total = walk.per_tile * walk.tiles;
    return walk;
}

struct WeightStream {
    uint32_t ring_begin, ring_end;  // shared-space address of this thread's 16 bytes (first half) of ring unit 0 / one past the last unit
    uint32_t head, tail;            // the same position in the unit to consume next / to request next
    uint32_t scale_offset;          // from there to this thread's scale word: 1024 + lane * 4 - lane * 16
    int units;                      // ring units of this warp (2..MAX_RING_UNITS, as shared memory allows)
    int used;                       // units requested and not yet consumed
    int in_flight;                  // items (copy groups) requested and not yet consumed
    // producer: the matrix being requested from, and the position in it
    int source_phase, rt, per_tile, remaining, gi;
    const uint4 *weights;           // the matrix, moved on by this thread's lane: + offset = its 16 bytes of the next block
    const uint32_t *scales;         // the scale pairs, moved on by lane / 4: + (offset >> 3) = this thread's pair of that block
    uint32_t offset;                // in 16-byte words; one block is 64 of them
    uint32_t step, tile_step;       // to the warp's next block inside a tile / to its first block of the CTA's next tile
    MatrixWalk following;           // the matrix after it (valid when has_following)
    bool has_following;
};

__device__ __forceinline__ void stream_start(WeightStream &stream, const MatrixWalk &walk, int phase) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    stream.source_phase = phase;
    stream.rt = walk.rt;
    stream.per_tile = walk.per_tile;
    stream.remaining = walk.total;
    stream.gi = 0;
    stream.weights = walk.matrix.weights + lane;
    stream.scales = walk.matrix.scales + (lane >> 2);
    stream.offset = (blockIdx.x * static_cast<uint32_t>(walk.matrix.groups) + warp) * walk.rt * 64u;
    stream.step = static_cast<uint32_t>(STACK_WARPS) * walk.rt * 64u;
    stream.tile_step = (gridDim.x * static_cast<uint32_t>(walk.matrix.groups) - (walk.per_tile - 1) * STACK_WARPS) * walk.rt * 64u;
}

// Requests the producer's next item of RT units (the ring has room and the matrix has items left).
template <int RT>
__device__ __forceinline__ void stream_issue_item(WeightStream &stream) {
    const uint4 *source = stream.weights + stream.offset;
    const uint32_t *scale_source = stream.scales + (stream.offset >> 3);
#pragma unroll
    for (int r = 0; r < RT; r++) {
        if (r == 0) {
            async_copy16<0, 0>(stream.tail, source);
            async_copy16<512, 512>(stream.tail, source);
            async_copy4<0>(stream.tail + stream.scale_offset, scale_source);
        } else {
            async_copy16<0, 1024>(stream.tail, source);
            async_copy16<512, 1536>(stream.tail, source);
            async_copy4<32>(stream.tail + stream.scale_offset, scale_source);
        }
        stream.tail += RING_UNIT_BYTES;
        if (stream.tail == stream.ring_end) stream.tail = stream.ring_begin;
    }
    async_commit();
    stream.used += RT;
    stream.in_flight++;
    stream.remaining--;
    // next block of this warp: 16 groups on, or the first group of the CTA's next tile
    uint32_t advance = stream.step;
    if (++stream.gi == stream.per_tile) {
        stream.gi = 0;
        advance = stream.tile_step;
    }
    stream.offset += advance;
}
__device__ __forceinline__ void stream_issue(WeightStream &stream) {
    if (stream.rt == 2) stream_issue_item<2>(stream);
    else stream_issue_item<1>(stream);
}

// Requests as many blocks as the ring has room for, moving on to the following matrix when this one is done.
__device__ __forceinline__ void stream_advance(WeightStream &stream) {
    while (true) {
        if (stream.remaining == 0) {
            if (!stream.has_following) break;
            stream_start(stream, stream.following, stream.source_phase + 1);
            stream.has_following = false;
            continue;
        }
        if (stream.units - stream.used < stream.rt) break;
        stream_issue(stream);
    }
}

// Asks the memory system to bring the CTA's tiles of a matrix into L2 (no registers or shared memory are tied
// up, nothing waits on it): issued one step ahead, so that HBM keeps streaming through the barriers, the staging
// and the attention of the step in between and the ring's copies then find their bytes in L2.
__device__ __forceinline__ void prefetch_l2(const void *address, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(__cvta_generic_to_global(address)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void prefetch_matrix_l2(const TiledInt4 &matrix, int rt) {
    constexpr uint32_t PIECE = 16384;
    const uint32_t tile_bytes = static_cast<uint32_t>(matrix.groups) * rt * 1024u, pieces = (tile_bytes + PIECE - 1) / PIECE;
    const int tiles = matrix.tiles > static_cast<int>(blockIdx.x)
                          ? (matrix.tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x)
                          : 0;
    for (uint32_t index = threadIdx.x; index < tiles * (pieces + 1); index += STACK_THREADS) {
        const uint32_t t = index / (pieces + 1), piece = index % (pieces + 1);
        const size_t tile = blockIdx.x + static_cast<size_t>(t) * gridDim.x;
        if (piece == pieces) {
            prefetch_l2(matrix.scales + tile * matrix.groups * rt * 8, static_cast<uint32_t>(matrix.groups) * rt * 32u);
        } else {
            const uint32_t offset = piece * PIECE, bytes = tile_bytes - offset < PIECE ? tile_bytes - offset : PIECE;
            prefetch_l2(reinterpret_cast<const uint8_t *>(matrix.weights + tile * matrix.groups * rt * 64) + offset, bytes);
        }
    }
}

// ------------------------------------------------------------------------------------------ activation staging

// A chunk is a uint4 of 8 consecutive bf16 of one lane; 16 consecutive chunks are one group of 128 columns.
// Chunk c of lane m -> fragment slot of thread (g = m, j) for word w, with group = c / 16, j = (c / 4) % 4,
// w = c % 4, is ((group * 4 + w) * staged + m) * 4 + j and holds (v0,v4) (v1,v5) (v2,v6) (v3,v7): the B operands of
// the two MMAs that consume nibble pairs (0,4) (1,5) and (2,6) (3,7) of the matching weight word.
__device__ __forceinline__ void stage_chunk(const StackSmem &sm, uint4 raw, bool active, int m, int chunk, int staged) {
    const int group = chunk >> 4, j = (chunk >> 2) & 3, word = chunk & 3;
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
    if (active && (chunk & 15) == 0) sm.correction[group * 8 + m] = -NIBBLE_BIAS * sum;  // the accumulation chains start from it
}

// Permutes [staged][width] bf16 rows into fragment order.  from_global: the rows were written by other CTAs of
// this launch and are read through L2; otherwise they are sm.rows.  Loads go out in batches of eight (two chunks of
// four lanes) before any of them is used: a pass costs one memory latency per batch, not one per chunk.
__device__ __forceinline__ void stage_rows(const StackSmem &sm, const uint16_t *x, bool from_global, int width, int staged) {
    const int per_lane = width >> 3;  // chunks of a lane, a multiple of 16
    const uint4 *source = from_global ? reinterpret_cast<const uint4 *>(x) : reinterpret_cast<const uint4 *>(sm.rows);
    for (int m0 = 0; m0 < staged; m0 += 4) {
        for (int base = 0; base < per_lane; base += STACK_THREADS * 2) {
            uint4 raw[2][4];
#pragma unroll
            for (int i = 0; i < 2; i++)
#pragma unroll
                for (int mm = 0; mm < 4; mm++) {
                    const int chunk = base + i * STACK_THREADS + threadIdx.x;
                    raw[i][mm] = make_uint4(0, 0, 0, 0);
                    if (chunk < per_lane && m0 + mm < staged) {
                        const uint4 *address = source + static_cast<size_t>(m0 + mm) * per_lane + chunk;
                        raw[i][mm] = from_global ? __ldcg(address) : *address;
                    }
                }
#pragma unroll
            for (int i = 0; i < 2; i++)
#pragma unroll
                for (int mm = 0; mm < 4; mm++) {
                    const int chunk = base + i * STACK_THREADS + threadIdx.x;
                    // uniform over the CTA: whole warps take part in the shuffles
                    if (base + i * STACK_THREADS < per_lane && m0 + mm < staged)
                        stage_chunk(sm, raw[i][mm], chunk < per_lane, m0 + mm, chunk < per_lane ? chunk : 0, staged);
                }
        }
    }
    for (int c = threadIdx.x; c < (width >> 7) * 8; c += STACK_THREADS)
        if ((c & 7) >= staged) sm.correction[c] = 0.0f;
    __syncthreads();
}

// rms_norm_bf16.comp.template:49-72 of every staged lane, straight into fragment order (each CTA repeats it:
// 8 KB per lane from L2).  A thread owns chunk t (and t + 512 when CHUNKS = 2) of each lane, four lanes at a time:
// one pass over registers for the sums of squares, one block-wide exchange, then normalise, round and permute.
template <int CHUNKS>  // chunks per thread and lane: width <= CHUNKS * 8 * STACK_THREADS
__device__ __forceinline__ void stage_normalised(const StackSmem &sm, const uint16_t *x, const uint16_t *weight, int width, int staged,
                                                 float eps, float offset) {
    const int per_lane = width >> 3, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint4 *source = reinterpret_cast<const uint4 *>(x);
    uint4 scale_words[CHUNKS];
#pragma unroll
    for (int c = 0; c < CHUNKS; c++) {
        const int chunk = threadIdx.x + c * STACK_THREADS;
        scale_words[c] = chunk < per_lane ? __ldg(reinterpret_cast<const uint4 *>(weight) + chunk) : make_uint4(0, 0, 0, 0);
    }
    for (int m0 = 0; m0 < staged; m0 += 4) {
        uint4 raw[4][CHUNKS];
#pragma unroll
        for (int mm = 0; mm < 4; mm++)
#pragma unroll
            for (int c = 0; c < CHUNKS; c++) {
                const int chunk = threadIdx.x + c * STACK_THREADS;
                raw[mm][c] = (m0 + mm < staged && chunk < per_lane) ? __ldcg(source + static_cast<size_t>(m0 + mm) * per_lane + chunk)
                                                                    : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
        for (int mm = 0; mm < 4; mm++) {
            float sum = 0.0f;
#pragma unroll
            for (int c = 0; c < CHUNKS; c++) {
                const uint32_t words[4] = {raw[mm][c].x, raw[mm][c].y, raw[mm][c].z, raw[mm][c].w};
#pragma unroll
                for (int w = 0; w < 4; w++) {
                    const float lo = bf16_lo(words[w]), hi = bf16_hi(words[w]);
                    sum = fmaf(lo, lo, sum);
                    sum = fmaf(hi, hi, sum);
                }
            }
            sum = warp_sum(sum);
            if (lane == 0) sm.partial[mm * STACK_WARPS + warp] = sum;
        }
        __syncthreads();
        // every warp adds up the 16 partials of the four lanes: lanes 8k .. 8k+7 of the warp take lane m0 + k
        float total = sm.partial[(lane >> 3) * STACK_WARPS + (lane & 7) * 2] + sm.partial[(lane >> 3) * STACK_WARPS + (lane & 7) * 2 + 1];
        total += __shfl_xor_sync(0xffffffffu, total, 1);
        total += __shfl_xor_sync(0xffffffffu, total, 2);
        total += __shfl_xor_sync(0xffffffffu, total, 4);
        // IEEE sqrt and divide, as a CPU evaluates 1/sqrt(v)
        const float my_inverse = 1.0f / sqrtf(total * (1.0f / static_cast<float>(width)) + eps);
#pragma unroll
        for (int mm = 0; mm < 4; mm++) {
            const float inv_rms = __shfl_sync(0xffffffffu, my_inverse, mm * 8);
#pragma unroll
            for (int c = 0; c < CHUNKS; c++) {
                const int chunk = threadIdx.x + c * STACK_THREADS;
                if (c * STACK_THREADS < per_lane && m0 + mm < staged) {  // uniform over the CTA
                    const uint32_t in[4] = {raw[mm][c].x, raw[mm][c].y, raw[mm][c].z, raw[mm][c].w};
                    const uint32_t sc[4] = {scale_words[c].x, scale_words[c].y, scale_words[c].z, scale_words[c].w};
                    uint32_t out[4];
#pragma unroll
                    for (int w = 0; w < 4; w++)
                        out[w] = pack_bf16(bf16_lo(in[w]) * inv_rms * (bf16_lo(sc[w]) + offset), bf16_hi(in[w]) * inv_rms * (bf16_hi(sc[w]) + offset));
                    stage_chunk(sm, make_uint4(out[0], out[1], out[2], out[3]), chunk < per_lane, m0 + mm, chunk < per_lane ? chunk : 0, staged);
                }
            }
        }
        if (m0 + 4 < staged) __syncthreads();  // sm.partial is rewritten for the next four lanes
    }
    for (int c = threadIdx.x; c < (width >> 7) * 8; c += STACK_THREADS)
        if ((c & 7) >= staged) sm.correction[c] = 0.0f;
    __syncthreads();
}

// ------------------------------------------------------------------------------------------ attention
// A team of four warps serves one context split (64 tokens) of one kv head for the Q = QL * GROUP <= 16 query
// vectors of QL consecutive lanes of a stream (append_gqa_attention_bf16.comp.template:217-339: f32 scores of
// bf16 q.k, f32 softmax, f32 p.v); warp w of the team takes tokens 16w .. 16w + 15 of the split.  Scores and p.v
// run on the tensor cores: q rows are the A operand of S = Q K^T, K rows the B operand (both read with 16-byte
// loads; the head dimension is permuted identically on both sides); the probabilities are re-used from the
// accumulator registers as the A operand of O = P V, split into a bf16 high and low part (p = hi + lo to 2^-17),
// and V is the B operand, its token pairs assembled with byte permutes.  The warps agree on the split's row
// maxima through shared memory, add up their partial outputs there, and the team writes one partial
// (unnormalised output, maximum, sum) to the scratch the merge step reads.

__device__ __forceinline__ void team_barrier(int barrier_id) { asm volatile("bar.sync %0, 128;" ::"r"(barrier_id) : "memory"); }

template <int HD>
__host__ __device__ constexpr size_t attention_team_bytes() {
    return (4 * 16 * HD + 2 * 4 * 16) * sizeof(float);  // partial outputs [warp][row][dim], maxima and sums [warp][row]
}

template <int HD, int GROUP, int QL>
__device__ __forceinline__ void attention_team_item(const uint16_t *__restrict__ q, const KvLayer &kv, const LaneTable &lanes_meta,
                                                    int lanes, int lanes_per_stream, int q_heads, float scale, int max_splits,
                                                    float *__restrict__ scratch, int kv_head, int split, int group_slot,
                                                    float *team_smem, int team_warp, int barrier_id) {
    constexpr int Q = QL * GROUP;
    constexpr int QW = HD / 32;                    // 16-byte pieces of a q / k row per thread
    constexpr int HALF = HD < 64 ? HD : 64;        // head dims handled per output pass
    constexpr int DPT = HALF / 8;                  // of which one thread column owns this many
    static_assert(Q <= 16 && HD % 32 == 0, "attention team shape");
    const int lane = threadIdx.x & 31, g = lane >> 2, j = lane & 3;
    float *partial_out = team_smem;                       // [4][16][HD]
    float *team_max = team_smem + 4 * 16 * HD;            // [4][16]
    float *team_sum = team_max + 4 * 16;                  // [4][16]
    const int groups_per_stream = (lanes_per_stream + QL - 1) / QL;
    const int stream_index = group_slot / groups_per_stream, group_index = group_slot % groups_per_stream;
    const int lane0 = stream_index * lanes_per_stream + group_index * QL;
    if (lane0 >= lanes) return;
    const int slot = lanes_meta.slot[lane0];
    if (slot < 0) return;
    const uint32_t capacity = kv.capacity;

    uint32_t newest = 0, tick_row[2] = {0xffffffffu, 0xffffffffu};
#pragma unroll
    for (int i = 0; i < QL; i++) {
        const bool valid = lane0 + i < lanes && group_index * QL + i < lanes_per_stream;
        const uint32_t tick = valid ? lanes_meta.position[lane0 + i] : 0xffffffffu;
        if (valid && tick > newest) newest = tick;
        if (g < Q && g / GROUP == i) tick_row[0] = tick;
        if (g + 8 < Q && (g + 8) / GROUP == i) tick_row[1] = tick;
    }
    const uint32_t tokens = newest + 1u < capacity ? newest + 1u : capacity;  // attended window of the newest lane
    const uint32_t first_tick = newest + 1u - tokens;
    const uint32_t begin = static_cast<uint32_t>(split) * 64u;
    if (begin >= tokens) return;  // the whole team leaves: nobody waits at the team barrier
    const int count = static_cast<int>(tokens - begin < 64u ? tokens - begin : 64u);
    const int token0 = 16 * team_warp;  // this warp's tokens of the split
    // ring index of the split's first token; element offset of token t's K (or V) row of this kv head
    const uint32_t ring_base = (first_tick + begin) % capacity;
    const int page_shift = (kv.page_tokens & (kv.page_tokens - 1)) == 0 ? __ffs(kv.page_tokens) - 1 : -1;
    const size_t half_page = static_cast<size_t>(kv.kv_heads) * kv.page_tokens * HD;
    auto row_offset = [&](int token, bool value) {
        uint32_t ring = ring_base + static_cast<uint32_t>(token);
        if (ring >= capacity) ring -= capacity;
        const int page = page_shift >= 0 ? static_cast<int>(ring >> page_shift) : static_cast<int>(ring / kv.page_tokens);
        const int within = page_shift >= 0 ? static_cast<int>(ring & (kv.page_tokens - 1)) : static_cast<int>(ring % kv.page_tokens);
        const int physical = kv.block_table[static_cast<size_t>(slot) * kv.pages_per_slot + page];
        return static_cast<size_t>(physical) * (2 * half_page) + (value ? half_page : 0) +
               (static_cast<size_t>(kv_head) * kv.page_tokens + within) * HD;
    };

    // ---- S = Q K^T for 16 tokens
    uint4 qf[2][QW];
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const int row = g + 8 * r;
        const bool valid = tick_row[r] != 0xffffffffu;
        const uint16_t *source = q + (static_cast<size_t>(lane0 + row / GROUP) * q_heads + kv_head * GROUP + row % GROUP) * HD + j * (HD / 4);
#pragma unroll
        for (int w = 0; w < QW; w++) qf[r][w] = valid ? __ldcg(reinterpret_cast<const uint4 *>(source) + w) : make_uint4(0, 0, 0, 0);
    }
    float s[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; nt++) {
        const int token = token0 + nt * 8 + g;
        uint4 kf[QW];
        if (token < count) {
            const uint16_t *krow = kv.pool + row_offset(token, false) + j * (HD / 4);
#pragma unroll
            for (int w = 0; w < QW; w++) kf[w] = __ldcg(reinterpret_cast<const uint4 *>(krow) + w);
        } else {
#pragma unroll
            for (int w = 0; w < QW; w++) kf[w] = make_uint4(0, 0, 0, 0);
        }
        s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
#pragma unroll
        for (int w = 0; w < QW; w++) {
            mma_bf16_16816(s[nt], qf[0][w].x, qf[1][w].x, qf[0][w].y, qf[1][w].y, kf[w].x, kf[w].y);
            mma_bf16_16816(s[nt], qf[0][w].z, qf[1][w].z, qf[0][w].w, qf[1][w].w, kf[w].z, kf[w].w);
        }
    }
    // V rows of this warp's tokens 2j, 2j+1, 2j+8, 2j+9 (requested now, used after the softmax)
    size_t v_offset[4];
#pragma unroll
    for (int t = 0; t < 4; t++) {
        const int token = token0 + 2 * j + (t & 1) + 8 * (t >> 1);
        v_offset[t] = token < count ? row_offset(token, true) : static_cast<size_t>(-1);
    }

    // ---- causal / ring mask, scale; the team's row maxima; probabilities
    float row_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; nt++)
#pragma unroll
        for (int c = 0; c < 4; c++) {
            const int token = token0 + nt * 8 + 2 * j + (c & 1);
            const uint32_t tick = tick_row[c >> 1], token_tick = first_tick + begin + token;
            const bool visible = token < count && tick != 0xffffffffu && token_tick <= tick && token_tick + capacity > tick;
            s[nt][c] = visible ? s[nt][c] * scale : -INFINITY;
            row_max[c >> 1] = fmaxf(row_max[c >> 1], s[nt][c]);
        }
#pragma unroll
    for (int r = 0; r < 2; r++) {
        row_max[r] = fmaxf(row_max[r], __shfl_xor_sync(0xffffffffu, row_max[r], 1));
        row_max[r] = fmaxf(row_max[r], __shfl_xor_sync(0xffffffffu, row_max[r], 2));
        if (j == 0) team_max[team_warp * 16 + g + 8 * r] = row_max[r];
    }
    team_barrier(barrier_id);
    float row_sum[2] = {0.0f, 0.0f};
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const int row = g + 8 * r;
        row_max[r] = fmaxf(fmaxf(team_max[row], team_max[16 + row]), fmaxf(team_max[32 + row], team_max[48 + row]));
        row_max[r] = fmaxf(row_max[r], -3.4028234663852886e38f);
    }
#pragma unroll
    for (int nt = 0; nt < 2; nt++)
#pragma unroll
        for (int c = 0; c < 4; c++) {
            s[nt][c] = s[nt][c] == -INFINITY ? 0.0f : expf(s[nt][c] - row_max[c >> 1]);
            row_sum[c >> 1] += s[nt][c];
        }
#pragma unroll
    for (int r = 0; r < 2; r++) {
        row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 1);
        row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 2);
        if (j == 0) team_sum[team_warp * 16 + g + 8 * r] = row_sum[r];
    }
    // probabilities as the A fragment of this warp's 16 tokens: high and low bf16 parts
    uint32_t ph[4], pl[4];
#pragma unroll
    for (int f = 0; f < 4; f++) {
        const float first = s[f >> 1][2 * (f & 1)], second = s[f >> 1][2 * (f & 1) + 1];
        ph[f] = pack_bf16(first, second);
        pl[f] = pack_bf16(first - bf16_lo(ph[f]), second - bf16_hi(ph[f]));
    }

    // ---- O = P V over the warp's tokens, HALF head dims per pass; thread column g owns dims DPT*g .. DPT*g+DPT-1
    float *mine = partial_out + static_cast<size_t>(team_warp) * 16 * HD;
#pragma unroll
    for (int pass = 0; pass < HD / HALF; pass++) {
        float o[DPT][4];
#pragma unroll
        for (int i = 0; i < DPT; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
        uint32_t v[4][DPT / 2];
#pragma unroll
        for (int t = 0; t < 4; t++) {
            if (v_offset[t] != static_cast<size_t>(-1)) {
                const uint16_t *vrow = kv.pool + v_offset[t] + pass * HALF + DPT * g;
                if (DPT == 8) {
                    const uint4 raw = __ldcg(reinterpret_cast<const uint4 *>(vrow));
                    v[t][0] = raw.x;
                    v[t][1] = raw.y;
                    v[t][DPT / 2 - 2] = raw.z;
                    v[t][DPT / 2 - 1] = raw.w;
                } else {
                    const uint2 raw = __ldcg(reinterpret_cast<const uint2 *>(vrow));
                    v[t][0] = raw.x;
                    v[t][DPT / 2 - 1] = raw.y;
                }
            } else {
#pragma unroll
                for (int w = 0; w < DPT / 2; w++) v[t][w] = 0u;
            }
        }
#pragma unroll
        for (int i = 0; i < DPT; i++) {
            const uint32_t selector = (i & 1) ? 0x7632u : 0x5410u;
            const uint32_t b0 = __byte_perm(v[0][i >> 1], v[1][i >> 1], selector), b1 = __byte_perm(v[2][i >> 1], v[3][i >> 1], selector);
            mma_bf16_16816(o[i], ph[0], ph[1], ph[2], ph[3], b0, b1);
            mma_bf16_16816(o[i], pl[0], pl[1], pl[2], pl[3], b0, b1);
        }
        // accumulator column 2j (+1) of output tile i is head dim DPT * (2j (+1)) + i of the pass
#pragma unroll
        for (int r = 0; r < 2; r++)
#pragma unroll
            for (int i = 0; i < DPT; i++) {
                mine[(g + 8 * r) * HD + pass * HALF + DPT * (2 * j) + i] = o[i][2 * r];
                mine[(g + 8 * r) * HD + pass * HALF + DPT * (2 * j + 1) + i] = o[i][2 * r + 1];
            }
    }
    team_barrier(barrier_id);
    // ---- the four partial outputs add up; warp w writes head dims [w * HD / 4, (w + 1) * HD / 4) of every row
    for (int index = lane; index < 16 * (HD / 4); index += 32) {
        const int row = index / (HD / 4), d = team_warp * (HD / 4) + index % (HD / 4);
        const int query_lane = lane0 + row / GROUP;  // rows beyond Q are padding
        const bool valid = row < Q && query_lane < lanes && group_index * QL + row / GROUP < lanes_per_stream;
        if (!valid) continue;
        const float sum = partial_out[row * HD + d] + partial_out[(16 + row) * HD + d] + partial_out[(32 + row) * HD + d] +
                          partial_out[(48 + row) * HD + d];
        float *out = scratch + ((static_cast<size_t>(query_lane) * q_heads + kv_head * GROUP + row % GROUP) * max_splits + split) * (HD + 2);
        out[d] = sum;
        if (d == 0) {
            out[HD] = fmaxf(fmaxf(fmaxf(team_max[row], team_max[16 + row]), fmaxf(team_max[32 + row], team_max[48 + row])), -3.4028234663852886e38f);
            out[HD + 1] = team_sum[row] + team_sum[16 + row] + team_sum[32 + row] + team_sum[48 + row];
        }
    }
    team_barrier(barrier_id);  // the team's shared arrays are free for its next item
}

// Log-sum-exp merge of the split partials of one (lane, q head) pair by one warp: lane s of the warp weighs
// split s (s + 32, ...), every lane owns HD / 32 consecutive output dims, and the weighted rows are summed in
// split order with four vector loads in flight.
template <int HD>
__device__ __forceinline__ void attention_merge_warp(const float *__restrict__ scratch, uint16_t *__restrict__ out, const KvLayer &kv,
                                                     const LaneTable &lanes_meta, int pair, int q_heads, int max_splits) {
    constexpr int VEC = HD / 32, STRIDE = HD + 2;
    const int lane_id = threadIdx.x & 31, lane = pair / q_heads;
    if (lanes_meta.slot[lane] < 0) return;
    const uint32_t tick = lanes_meta.position[lane];
    const uint32_t tokens = tick + 1u < kv.capacity ? tick + 1u : kv.capacity;
    int splits = static_cast<int>((tokens + 63u) / 64u);
    if (splits > max_splits) splits = max_splits;
    const float *base = scratch + static_cast<size_t>(pair) * max_splits * STRIDE;
    float maximum = -3.4028234663852886e38f;
    for (int s = lane_id; s < splits; s += 32) maximum = fmaxf(maximum, __ldcg(base + static_cast<size_t>(s) * STRIDE + HD));
    maximum = warp_max(maximum);
    float denominator = 0.0f, acc[VEC];
#pragma unroll
    for (int v = 0; v < VEC; v++) acc[v] = 0.0f;
    for (int s0 = 0; s0 < splits; s0 += 32) {
        float weight = 0.0f;
        if (s0 + lane_id < splits) {
            weight = expf(__ldcg(base + static_cast<size_t>(s0 + lane_id) * STRIDE + HD) - maximum);
            denominator += __ldcg(base + static_cast<size_t>(s0 + lane_id) * STRIDE + HD + 1) * weight;
        }
        const int end = splits - s0 < 32 ? splits - s0 : 32;
        for (int s = 0; s < end; s += 4) {
            float part[4][VEC];
#pragma unroll
            for (int u = 0; u < 4; u++)
#pragma unroll
                for (int v = 0; v < VEC; v++)
                    part[u][v] = s + u < end ? __ldcg(base + static_cast<size_t>(s0 + s + u) * STRIDE + lane_id * VEC + v) : 0.0f;
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const float w = __shfl_sync(0xffffffffu, weight, (s + u) & 31);
#pragma unroll
                for (int v = 0; v < VEC; v++) acc[v] += part[u][v] * (s + u < end ? w : 0.0f);
            }
        }
    }
    denominator = warp_sum(denominator);
#pragma unroll
    for (int v = 0; v < VEC; v++)
        out[static_cast<size_t>(pair) * HD + lane_id * VEC + v] =
            static_cast<uint16_t>(f32_to_bf16_bits(denominator == 0.0f ? 0.0f : acc[v] / denominator));
}

// ------------------------------------------------------------------------------------------ the kernel

struct StackArgs {
    const StackLayer *layers;
    int layer_count;
    StackShape shape;
    StackBuffers buffers;
    LaneTable lanes_meta;
    int lanes, lanes_per_stream, split_tokens, max_splits;
    int ring_units, l2_prefetch;
    const StackTp *tp;  // device copy of the exchange description, or nullptr (single GPU)
    int tp_size;
};

struct StackSmemLayout {
    size_t fragments, rows, correction, reduce, partial, ring, total;
};
__host__ __device__ inline StackSmemLayout stack_smem_layout(const StackShape &shape, int staged, int ring_units) {
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
    layout.ring = layout.partial + 8 * STACK_WARPS * sizeof(float);
    layout.total = layout.ring + static_cast<size_t>(STACK_WARPS) * ring_units * RING_UNIT_BYTES;
    const size_t attention = 4 * (4 * 16 * static_cast<size_t>(shape.head_width) + 2 * 4 * 16) * sizeof(float);  // four attention teams
    if (attention > layout.total) layout.total = attention;
    return layout;
}

// One 16x128 block of the ring against the staged activations: eight MMAs over bf16 (16 + q) in two accumulation
// chains.  The first chain starts from -24 * sum(x) of the group (`negative_bias`, per lane), which takes the
// 16 + 8 offset of the nibbles out again; the sum of the chains is the block's product.
__device__ __forceinline__ void unit_products(uint32_t mine, const uint4 (&b)[4], float2 negative_bias, float (&c)[4]) {
    const uint4 first = shared_load16<0>(mine);
    const uint4 second = shared_load16<512>(mine);
    const uint32_t wa[4] = {first.x, first.y, first.z, first.w};
    const uint32_t wb[4] = {second.x, second.y, second.z, second.w};
    float even[4] = {negative_bias.x, negative_bias.y, negative_bias.x, negative_bias.y}, odd[4];
#pragma unroll
    for (int word = 0; word < 4; word++) {
        mma_bf16_16816(even, biased_pair<0>(wa[word]), biased_pair<0>(wb[word]), biased_pair<1>(wa[word]), biased_pair<1>(wb[word]), b[word].x,
                       b[word].y);
        if (word == 0)
            mma_bf16_16816_first(odd, biased_pair<2>(wa[word]), biased_pair<2>(wb[word]), biased_pair<3>(wa[word]), biased_pair<3>(wb[word]),
                                 b[word].z, b[word].w);
        else
            mma_bf16_16816(odd, biased_pair<2>(wa[word]), biased_pair<2>(wb[word]), biased_pair<3>(wa[word]), biased_pair<3>(wb[word]), b[word].z,
                           b[word].w);
    }
#pragma unroll
    for (int i = 0; i < 4; i++) c[i] = even[i] + odd[i];
}

// The block's two scales (rows g and g + 8).
__device__ __forceinline__ void unit_accumulate(uint32_t scales, const float (&c)[4], float (&acc)[4]) {
    const float sa = __uint_as_float(scales << 16), sb = __uint_as_float(scales & 0xffff0000u);
    acc[0] = fmaf(sa, c[0], acc[0]);
    acc[1] = fmaf(sa, c[1], acc[1]);
    acc[2] = fmaf(sb, c[2], acc[2]);
    acc[3] = fmaf(sb, c[3], acc[3]);
}

// A tile's items of this warp (RT ring units each): wait for the item's copies, issue its MMAs, put the freed ring
// units back to work while the tensor pipe runs, then fold the products into the tile's accumulators.
// xitem / bias_item: shared-space addresses of the thread's fragments and bias pair of the warp's first group.
template <int RT>
__device__ __forceinline__ void tile_items(WeightStream &stream, int items, uint32_t xitem, uint32_t bias_item, uint32_t word_stride,
                                           float (&acc)[2][4]) {
    const uint32_t item_stride = STACK_WARPS * 4 * word_stride;
    for (int gi = 0; gi < items; gi++) {
        uint4 b[4];
        b[0] = shared_load16<0>(xitem);
        b[1] = shared_load16<0>(xitem + word_stride);
        b[2] = shared_load16<0>(xitem + 2 * word_stride);
        b[3] = shared_load16<0>(xitem + 3 * word_stride);
        const float2 negative_bias = shared_load_float2(bias_item);
        xitem += item_stride;
        bias_item += STACK_WARPS * 8 * sizeof(float);
        async_wait_oldest(stream.in_flight);
        stream.in_flight--;
        float c[RT][4];
        uint32_t scales[RT];
#pragma unroll
        for (int r = 0; r < RT; r++) {
            scales[r] = shared_load4(stream.head + stream.scale_offset);
            unit_products(stream.head, b, negative_bias, c[r]);
            stream.head += RING_UNIT_BYTES;
            if (stream.head == stream.ring_end) stream.head = stream.ring_begin;
        }
        stream.used -= RT;
        if (stream.remaining > 0 && stream.rt == RT) stream_issue_item<RT>(stream);  // the freed units go straight back to work
        else stream_advance(stream);
#pragma unroll
        for (int r = 0; r < RT; r++) unit_accumulate(scales[r], c[r], acc[r]);
    }
}

template <int GROUP>
struct AttentionTeam {
    static constexpr int QL = GROUP >= 8 ? 2 : (GROUP >= 4 ? 4 : (16 / GROUP > 8 ? 8 : 16 / GROUP));
};

// EXCHANGE: the tensor-parallel form (o and down leave partial sums that are exchanged between the ranks).
template <int HD, int GROUP, bool EXCHANGE>
__global__ void __launch_bounds__(STACK_THREADS, 1) decode_stack_kernel(const StackArgs a) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    constexpr int QL = AttentionTeam<GROUP>::QL;
    const StackShape &shape = a.shape;
    const int lanes = a.lanes, staged = lanes < 8 ? lanes : 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, j = lane & 3;
    const StackSmemLayout layout = stack_smem_layout(shape, staged, a.ring_units);
    StackSmem sm;
    sm.fragments = reinterpret_cast<uint4 *>(smem_raw + layout.fragments);
    sm.rows = reinterpret_cast<uint16_t *>(smem_raw + layout.rows);
    sm.correction = reinterpret_cast<float *>(smem_raw + layout.correction);
    sm.reduce = reinterpret_cast<float *>(smem_raw + layout.reduce);
    sm.partial = reinterpret_cast<float *>(smem_raw + layout.partial);
    sm.ring = smem_raw + layout.ring;

    const int q_width = shape.q_heads * HD, q_tiles = q_width >> 4, k_tiles = (shape.kv_heads * HD) >> 4;
    unsigned int target = 0;
    constexpr bool exchanging = EXCHANGE;
    unsigned long long exchange_target = 0ull;  // exchanges done so far, earlier launches included
    float *exchange_mine = nullptr;
    if constexpr (EXCHANGE) {
        exchange_target = a.tp->counter[a.tp->rank][TP_WORD_CONSUMED];
        exchange_mine = a.tp->exchange[a.tp->rank];
    }
    int exchange_parity = 0;
    unsigned int *counter = a.buffers.barrier;
    int *error_flag = a.buffers.error_flag;
    int parity = 0, phase = 0;
    WeightStream stream;
    stream.ring_begin = static_cast<uint32_t>(__cvta_generic_to_shared(sm.ring + static_cast<size_t>(warp) * a.ring_units * RING_UNIT_BYTES + lane * 16));
    stream.ring_end = stream.ring_begin + a.ring_units * RING_UNIT_BYTES;
    stream.head = stream.tail = stream.ring_begin;
    stream.scale_offset = 1024 + lane * 4 - lane * 16;
    stream.units = a.ring_units;
    stream.used = 0;
    stream.rt = 1;
    stream.per_tile = 0;
    stream.gi = 0;
    stream.in_flight = 0;
    stream.has_following = false;
    stream.source_phase = -1;
    stream.remaining = 0;
    stream.weights = nullptr;
    stream.scales = nullptr;
    stream.offset = stream.step = stream.tile_step = 0;

    auto stamp = [&](int layer, int index) {
        if (a.buffers.timing != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            a.buffers.timing[layer * 32 + index] = now;
        }
    };
    // Epilogue roles: thread t < 128 finishes output (high = t & 1, lane m = (t >> 1) & 7, row = (t >> 4) + 8 * high)
    // of a tile's 16 rows x 8 lanes, so the rotary partner rows r and r + 8 of a lane sit in neighbouring threads.
    // Only four warps do this; the other twelve go straight on to the next tile's blocks.
    const int epilogue_m = (threadIdx.x >> 1) & 7, epilogue_row = (threadIdx.x >> 4) + 8 * (threadIdx.x & 1);
    const bool epilogue_active = threadIdx.x < 128 && epilogue_m < lanes;
    // per-lane constants of the epilogue: position, rotary table row, and the lane's KV row inside a page (the
    // block table is shared by all layers)
    uint32_t lane_position = 0;
    const uint32_t *rope_row = shape.rope_table;
    size_t kv_token_base = 0;
    bool kv_writable = false;
    if (threadIdx.x < 128 && epilogue_m < lanes) {
        lane_position = a.lanes_meta.position[epilogue_m];
        rope_row = shape.rope_table + static_cast<size_t>(lane_position % shape.rope_positions) * (HD >> 1);
        const KvLayer &kv0 = a.layers[0].kv;
        const int slot = a.lanes_meta.slot[epilogue_m];
        if (slot >= 0 && kv0.capacity != 0) {
            const uint32_t ring = lane_position % kv0.capacity;
            const int physical = kv0.block_table[static_cast<size_t>(slot) * kv0.pages_per_slot + ring / kv0.page_tokens];
            kv_token_base = static_cast<size_t>(physical) * 2 * kv0.kv_heads * kv0.page_tokens * HD + static_cast<size_t>(ring % kv0.page_tokens) * HD;
            kv_writable = true;
        }
    }
    const int ge = g < staged ? g : 0;  // lanes beyond the batch recompute lane 0; their results are dropped
    const uint32_t xlane = static_cast<uint32_t>(__cvta_generic_to_shared(sm.fragments + ge * 4 + j));
    const uint32_t bias_lane = static_cast<uint32_t>(__cvta_generic_to_shared(sm.correction + 2 * j));
    const uint32_t word_stride = static_cast<uint32_t>(staged) * 4 * sizeof(uint4);

    for (int layer = 0; layer < a.layer_count; layer++) {
        const StackLayer *spec = a.layers + layer;
        const KvLayer kv = spec->kv;
        for (int step = 0; step < 4; step++, phase++) {
            // ---- the matrix of this step, and the one whose first blocks may be requested while this one drains
            TiledInt4 matrix, next_matrix;
            int rt = 1, next_rt = 1;
            bool has_next = true;
            if (step == 0) {
                matrix = spec->qkv;
                next_matrix = matrix;
                has_next = false;  // attention sits in between; the o projection is requested after it
            } else if (step == 1) {
                matrix = spec->o;
                next_matrix = spec->gate_up;
                next_rt = 2;
            } else if (step == 2) {
                matrix = spec->gate_up;
                rt = 2;
                next_matrix = spec->down;
            } else {
                matrix = spec->down;
                has_next = layer + 1 < a.layer_count;
                next_matrix = has_next ? a.layers[layer + 1].qkv : matrix;
            }
            const MatrixWalk walk = walk_of(matrix, rt);
            if (stream.source_phase != phase) stream_start(stream, walk, phase);
            stream.has_following = has_next;
            if (has_next) stream.following = walk_of(next_matrix, next_rt);
            stream_advance(stream);
            // the matrix after this one goes to L2 now (the gate/up pair already while attention runs)
            if (!a.l2_prefetch) {
            } else if (step == 0) {
                prefetch_matrix_l2(spec->o, 1);
                prefetch_matrix_l2(spec->gate_up, 2);
            } else if (step == 2) {
                prefetch_matrix_l2(spec->down, 1);
            } else if (step == 3 && layer + 1 < a.layer_count) {
                prefetch_matrix_l2(a.layers[layer + 1].qkv, 1);
            }
            stamp(layer, 4 * step);

            // ---- activations of this step into fragment order
            if (step == 0 || step == 2) {
                const uint16_t *norm_weight = step == 0 ? spec->input_norm : spec->post_norm;
                if (shape.hidden <= 8 * STACK_THREADS)
                    stage_normalised<1>(sm, a.buffers.hidden, norm_weight, shape.hidden, staged, shape.eps, shape.norm_offset);
                else
                    stage_normalised<2>(sm, a.buffers.hidden, norm_weight, shape.hidden, staged, shape.eps, shape.norm_offset);
                if (step == 2) stamp(layer, 16);
            } else if (step == 1) {
                stage_rows(sm, a.buffers.attention_out, true, q_width, staged);
            } else {
                stage_rows(sm, a.buffers.activation, true, shape.ffn, staged);
            }
            stamp(layer, 4 * step + 1);

            // ---- the CTA's tiles: every warp takes each 16th group of K, then the tile is reduced and finished
            float acc[2][4];
#pragma unroll
            for (int r = 0; r < 2; r++) acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.0f;
            int tile = blockIdx.x;
            for (int t = 0; t < walk.tiles; t++, tile += gridDim.x) {
                // what the epilogue needs from memory is requested before the tile's arithmetic
                uint32_t payload = 0;
                if (epilogue_active) {
                    if (step == 0) {
                        if (tile < q_tiles + k_tiles) {
                            const int local = tile < q_tiles ? tile : tile - q_tiles;
                            payload = __ldg(rope_row + 8 * (local % (HD >> 4)) + (epilogue_row & 7));
                        }
                    } else if (step != 2 && !exchanging) {
                        payload = __ldcg(a.buffers.hidden + static_cast<size_t>(epilogue_m) * shape.hidden + tile * 16 + epilogue_row);
                    }
                }
                const uint32_t xitem = xlane + warp * 4 * word_stride;  // fragments of group `warp`, then 16 groups on per item
                const uint32_t bias_item = bias_lane + warp * 8 * sizeof(float);
                if (rt == 2) tile_items<2>(stream, walk.per_tile, xitem, bias_item, word_stride, acc);
                else tile_items<1>(stream, walk.per_tile, xitem, bias_item, word_stride, acc);
                float *mine = sm.reduce + static_cast<size_t>((parity * STACK_WARPS + warp) * 32) * 8;
#pragma unroll
                for (int r = 0; r < 2; r++) {
                    if (r < rt) {
                        *reinterpret_cast<float2 *>(mine + (r * 16 + g) * 8 + 2 * j) = make_float2(acc[r][0], acc[r][1]);
                        *reinterpret_cast<float2 *>(mine + (r * 16 + g + 8) * 8 + 2 * j) = make_float2(acc[r][2], acc[r][3]);
                    }
                    acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.0f;
                }
                __syncthreads();
                if (threadIdx.x < 128) {  // whole warps: the q/k epilogue exchanges partner rows by shuffle
                    const float *src = sm.reduce + static_cast<size_t>(parity * STACK_WARPS * 32 + epilogue_row) * 8 + epilogue_m;
                    float first = 0.0f, second = 0.0f;
#pragma unroll
                    for (int w = 0; w < STACK_WARPS; w++) {
                        first += src[w * 32 * 8];
                        if (rt == 2) second += src[(w * 32 + 16) * 8];
                    }
                    if (step == 0) {
                        // q / k: rotary_bf16.comp.template:99-109 (non-interleaved, rotary width = head width, five bf16
                        // roundings); k and v go into the lane's KV page (append_gqa_attention_bf16.comp.template:189-215)
                        const float mine_value = round_bf16(first);
                        const float partner = __shfl_xor_sync(0xffffffffu, mine_value, 1);  // the row 8 further (or 8 back)
                        if (epilogue_active) {
                            const size_t kv_half = static_cast<size_t>(kv.kv_heads) * kv.page_tokens * HD;
                            if (tile < q_tiles + k_tiles) {
                                const bool is_q = tile < q_tiles, high = epilogue_row >= 8;
                                const int local = is_q ? tile : tile - q_tiles;
                                const int head = local / (HD >> 4), d = 8 * (local % (HD >> 4)) + (epilogue_row & 7) + (high ? HD / 2 : 0);
                                const float cosine = bf16_lo(payload), sine = bf16_hi(payload);
                                // d < half: x cos + (-x[d + half]) sin;  d >= half: x cos + x[d - half] sin
                                const float other = high ? partner : -partner;
                                const uint16_t value = static_cast<uint16_t>(f32_to_bf16_bits(round_bf16(mine_value * cosine) + round_bf16(other * sine)));
                                if (is_q) a.buffers.q[(static_cast<size_t>(epilogue_m) * shape.q_heads + head) * HD + d] = value;
                                else if (kv_writable) kv.pool[kv_token_base + static_cast<size_t>(head) * kv.page_tokens * HD + d] = value;
                            } else if (kv_writable) {
                                const int index = (tile - q_tiles - k_tiles) * 16 + epilogue_row;
                                kv.pool[kv_token_base + kv_half + static_cast<size_t>(index / HD) * kv.page_tokens * HD + index % HD] =
                                    static_cast<uint16_t>(f32_to_bf16_bits(first));
                            }
                        }
                    } else if (epilogue_active) {
                        if (step == 2) {
                            // silu_multiply_bf16.comp.template:30-52: bf16(silu_bf16(bf16 gate) * bf16 up)
                            a.buffers.activation[static_cast<size_t>(epilogue_m) * shape.ffn + tile * 16 + epilogue_row] =
                                static_cast<uint16_t>(f32_to_bf16_bits(rounded_silu(round_bf16(first)) * round_bf16(second)));
                        } else if constexpr (EXCHANGE) {
                            // this rank's share of the sum over K, unrounded, into its exchange buffer (the others fetch it)
                            exchange_mine[(static_cast<size_t>(exchange_parity) * 8 + epilogue_m) * shape.hidden + tile * 16 + epilogue_row] = first;
                        } else {
                            // linear + residual_add (add_bf16.comp.template:17-24): bf16(bf16(product) + residual), in place
                            a.buffers.hidden[static_cast<size_t>(epilogue_m) * shape.hidden + tile * 16 + epilogue_row] =
                                static_cast<uint16_t>(f32_to_bf16_bits(round_bf16(first) + bf16_bits_to_f32(payload)));
                        }
                    }
                }
                parity ^= 1;
            }
            stamp(layer, 4 * step + 2);
            if constexpr (EXCHANGE) {
              if (step == 1 || step == 3) {
                exchange_barrier(*a.tp, exchange_target, error_flag);
                reduce_exchanged(*a.tp, exchange_parity, a.buffers.hidden, lanes, shape.hidden);
                exchange_parity ^= 1;
              }
            }
            grid_barrier(counter, target, error_flag);
            stamp(layer, 4 * step + 3);

            if (step == 0) {
                // ---- attention: (kv head, split, stream x lane group) items, one team of four warps each, spread
                // over the SMs first; the teams' shared arrays reuse the staging area (nothing is staged right now)
                const int streams = lanes / a.lanes_per_stream;
                const int group_slots = streams * ((a.lanes_per_stream + QL - 1) / QL);
                const int total = shape.kv_heads * a.max_splits * group_slots;
                const int team = warp >> 2;
                float *team_smem = reinterpret_cast<float *>(smem_raw + static_cast<size_t>(team) * attention_team_bytes<HD>());
                for (int item = blockIdx.x + gridDim.x * team; item < total; item += gridDim.x * 4) {
                    const int kv_head = item % shape.kv_heads, rest = item / shape.kv_heads;
                    attention_team_item<HD, GROUP, QL>(a.buffers.q, kv, a.lanes_meta, lanes, a.lanes_per_stream, shape.q_heads,
                                                       shape.attention_scale, a.max_splits, a.buffers.attention_scratch, kv_head,
                                                       rest % a.max_splits, rest / a.max_splits, team_smem, warp & 3, 1 + team);
                }
                __syncthreads();  // the ring shares bytes with the teams' arrays
                stamp(layer, 17);
                // the o projection's first blocks stream while the grid meets and merges
                stream_start(stream, walk_of(spec->o, 1), phase + 1);
                stream.has_following = false;
                stream_advance(stream);
                grid_barrier(counter, target, error_flag);
                stamp(layer, 18);
                const int pairs = lanes * shape.q_heads;
                for (int pair = blockIdx.x + gridDim.x * warp; pair < pairs; pair += gridDim.x * STACK_WARPS)
                    attention_merge_warp<HD>(a.buffers.attention_scratch, a.buffers.attention_out, kv, a.lanes_meta, pair, shape.q_heads,
                                             a.max_splits);
                stamp(layer, 19);
                grid_barrier(counter, target, error_flag);
            }
        }
    }

    // The last CTA to leave rearms the barrier words for the next launch (every CTA has passed its last barrier
    // before it counts itself out).
    if (threadIdx.x == 0) {
        const unsigned int gone = atomicAdd(counter + 1, 1u);
        if (gone == gridDim.x - 1) {
            counter[0] = 0u;
            counter[1] = 0u;
            if constexpr (EXCHANGE) a.tp->counter[a.tp->rank][TP_WORD_CONSUMED] = exchange_target;  // the next launch counts on from here
            __threadfence();
        }
    }
}

template <int HD, int GROUP, bool EXCHANGE>
cudaError_t launch_instance_of(const StackArgs &args, size_t smem, cudaStream_t stream) {
    static int configured_device = -1, sm_count = 0;
    int device = 0;
    cudaError_t status = cudaGetDevice(&device);
    if (status != cudaSuccess) return status;
    if (configured_device != device) {
        status = cudaFuncSetAttribute(decode_stack_kernel<HD, GROUP, EXCHANGE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
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
    return cudaLaunchKernelEx(&config, decode_stack_kernel<HD, GROUP, EXCHANGE>, args);
}

template <int HD, int GROUP>
cudaError_t launch_instance(const StackArgs &args, size_t smem, cudaStream_t stream) {
    return args.tp_size > 1 ? launch_instance_of<HD, GROUP, true>(args, smem, stream) : launch_instance_of<HD, GROUP, false>(args, smem, stream);
}

bool instance_smem(const StackShape &shape, int lanes, size_t *bytes, int *ring_units) {
    const int group = shape.kv_heads > 0 ? shape.q_heads / shape.kv_heads : 0;
    const bool built = (shape.head_width == 128 && (group == 4 || group == 8)) || (shape.head_width == 64 && group == 4) ||
                       (shape.head_width == 32 && group == 2);
    if (!built) return false;
    // the deepest ring the 227 KB of shared memory leave room for (an even count: a gate/up item takes two units)
    int units = MAX_RING_UNITS;
    static const char *forced = getenv("NERVE_B200_STACK_RING");
    if (forced != nullptr && atoi(forced) >= 2 && atoi(forced) <= MAX_RING_UNITS) units = atoi(forced) & ~1;
    while (units > 2 && stack_smem_layout(shape, lanes < 8 ? lanes : 8, units).total > 227 * 1024) units -= 2;
    *bytes = stack_smem_layout(shape, lanes < 8 ? lanes : 8, units).total;
    if (ring_units) *ring_units = units;
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
    if (shape.hidden > 2 * 8 * STACK_THREADS || shape.hidden % 128 != 0 || shape.ffn % 128 != 0 || (shape.q_heads * shape.head_width) % 128 != 0) return false;
    if (!instance_smem(shape, lanes, &bytes, nullptr)) return false;
    if (bytes > 227 * 1024) return false;
    if (smem_bytes) *smem_bytes = bytes;
    return true;
}

cudaError_t launch_decode_stack(const StackLayer *layers_device, int layer_count, const StackShape &shape,
                                const StackBuffers &buffers, const LaneTable &lanes_meta, int lanes, int lanes_per_stream,
                                int split_tokens, int max_splits, cudaStream_t stream, const StackTp *tp_device, int tp_size) {
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
    if (tp_size < 1 || tp_size > STACK_TP_MAX_RANKS || (tp_size > 1 && (tp_device == nullptr || shape.hidden % 4 != 0))) return cudaErrorInvalidValue;
    args.tp = tp_size > 1 ? tp_device : nullptr;
    args.tp_size = tp_size;
    instance_smem(shape, lanes, &smem, &args.ring_units);
    static const char *prefetch = getenv("NERVE_B200_STACK_L2_PREFETCH");
    args.l2_prefetch = (prefetch != nullptr && prefetch[0] == '1') ? 1 : 0;  // off: the tile loops are not HBM-bound (yet)
    const int group = shape.q_heads / shape.kv_heads;
    if (shape.head_width == 128 && group == 4) return launch_instance<128, 4>(args, smem, stream);
    if (shape.head_width == 128 && group == 8) return launch_instance<128, 8>(args, smem, stream);
    if (shape.head_width == 64 && group == 4) return launch_instance<64, 4>(args, smem, stream);
    return launch_instance<32, 2>(args, smem, stream);
}

}  // namespace nerve

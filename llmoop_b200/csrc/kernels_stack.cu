// Persistent decode stack: one cooperative launch runs every layer of a dense INT4 g128 Llama-style stack
// (rms_norm, q/k/v, RoPE, KV append, attention, o + residual, rms_norm, gate/up + SiLU, down + residual:
// the kernel list of one reference layer component, runtime-rs/shaders/*.comp.template) for a batch of at most
// 8 lanes - the verify batch and the draft / single-tick steps of the speculative decode cycle.
//
// Why one launch: at these batch sizes a layer is ~112 MB of weights (~17 us of HBM time) cut into a dozen
// dependent steps; as separate kernels every step pays a launch, a pipeline fill and a drain.  Here one CTA per
// SM stays resident and the weight stream never stops for a step boundary:
//
//  * weights: at mount every matrix is rewritten as one contiguous byte stream per CTA, in exactly the order the
//    CTA consumes it (see stack_schedule in kernels.cuh).  A stream is a sequence of stages; a stage is one
//    16x128 block of packed nibbles (1 KB) plus its 32 bytes of scales for each of up to 16 warps.
//  * a producer thread (warp 16) walks the CTA's stages of all matrices of all layers and brings them into a ring
//    in shared memory with one bulk asynchronous copy per stage (mbarrier transaction counts; no cluster forms),
//    as far ahead as the ring allows - through the grid barriers, the attention step and the epilogues - and asks
//    L2 for the stages after those (cp.async.bulk.prefetch.L2) so that HBM keeps streaming while the SMs wait on
//    one another.
//  * 16 consumer warps: a CTA works on all its tiles of a matrix at once - warp w owns tile slot w / W and every
//    W-th block of K - so a matrix costs one cross-warp reduction and one epilogue pass per CTA instead of one per
//    tile.  Nibbles become exact fp16 (q - 8) operands (lop3 into the mantissa of 1024, one fp16 subtract or fma),
//    eight mma.sync m16n8k16 per block accumulate in f32, the group scale multiplies the block's f32 product as in
//    linear_int4_ct.comp.template:80-150.
//  * activations: the inputs of q/k/v and gate/up are normalised (rms_norm_bf16.comp.template:49-72) by every CTA
//    into shared memory in mma B-fragment order; the inputs of o and down are written by their producers
//    (attention merge, SiLU epilogue) to global memory already in fragment order and ride the ring, one slice per
//    stage, once the grid barrier in front of the step has opened.
//  * attention: a team of four warps per (kv head, 64-token split, lane group) on the tensor cores (query rows in
//    shared memory, K and V rows in registers, all loads of an item requested before its arithmetic); the team that
//    completes a kv head's last split queues the merge, and after its items the CTA's sixteen warps merge one
//    (lane, q head) row each - no grid barrier between the splits and their merge.  Lane groups of more than 32
//    splits are merged in two levels (ranges of 32 splits spread over every warp of the grid, then the ranges of a
//    row by one warp), with a grid barrier before each level.
//  * code that runs once per layer (staging, attention, merge, epilogues) is kept short and free of re-read state:
//    such straight-line code was measured at about 0.27 us per KB of instructions on this kernel (instruction
//    fetch, not arithmetic), and a value behind a reference is read again after every ordered load.
//  * tensor parallelism (the EXCHANGE instances): o and down push their f32 partial sums, tagged with the exchange
//    number in the same 8-byte store, into every peer's inbox over NVLink; the owner of an output element waits
//    for the peers' words in its own memory and adds them in rank order.  No barrier crosses the link.
//
// Every wait is bounded: when a bound expires the kernel sets the error word and leaves.
#include <cuda_fp16.h>

#include <cstdlib>

#include "common.cuh"
#include "kernels.cuh"

namespace nerve {

namespace {

constexpr int CONSUMER_WARPS = 16;
constexpr int CONSUMER_THREADS = CONSUMER_WARPS * 32;
constexpr int STACK_THREADS = CONSUMER_THREADS + 128;  // + the producer warps (registers are allotted four warps at a time)
constexpr int UNIT_BYTES = 1024;                      // packed nibbles of a 16x128 block
constexpr int UNIT_SCALE_BYTES = 32;                  // its eight scale pairs
constexpr int UNIT_TOTAL = UNIT_BYTES + UNIT_SCALE_BYTES;
constexpr int STAGE_WEIGHT_BYTES = 16 * UNIT_TOTAL;   // weight part of a ring stage (16 896 bytes)
constexpr int MAX_STAGES = 16;
constexpr unsigned int BARRIER_SPIN_LIMIT = 1u << 20;
constexpr unsigned int PIPE_SPIN_LIMIT = 1u << 18;  // attempts of about 20 us each at most
constexpr unsigned int OPEN_SPIN_LIMIT = 1u << 28;  // polls of the barrier count by the slice producer: it has to outlast the consumers' own waits
constexpr int BARRIERS_PER_LAYER = 5;  // after q/k/v, attention, o, gate/up, down
constexpr int ARRIVAL_WORDS_OFFSET = 16;  // attention arrival counters sit behind the two barrier words

// ------------------------------------------------------------------------------------------ per-CTA streams

struct RelayoutArgs {
    RelayoutSegment segment[3];
    int first_tile[4];
    int count;
    int pair;
    int k;
    MatrixSchedule schedule;
};

// Block (stage, cta) writes one stage of one CTA's stream: the present units' nibbles, then their scale pairs.
__global__ void int4_cta_stream_kernel(const RelayoutArgs args, uint8_t *__restrict__ out) {
    const MatrixSchedule &s = args.schedule;
    const int cta = blockIdx.y, stage = blockIdx.x;
    const int here = stack_cta_tiles(s, cta);
    const int pass = stage / s.steps, step = stage % s.steps;
    int present = here - pass * s.slots;
    if (present <= 0) return;
    if (present > s.slots) present = s.slots;
    const int groups = args.k >> 7;
    uint8_t *base = out + stack_cta_offset(s, cta) + static_cast<size_t>(pass) * s.slots * s.width * s.steps * UNIT_TOTAL +
                    static_cast<size_t>(step) * present * s.width * UNIT_TOTAL;
    uint4 *weights_out = reinterpret_cast<uint4 *>(base);
    uint32_t *scales_out = reinterpret_cast<uint32_t *>(base + static_cast<size_t>(present) * s.width * UNIT_BYTES);
    auto locate = [&](int unit_in_stage, int &group, int &which, int &local_tile) {
        const int slot = unit_in_stage / s.width, i = unit_in_stage % s.width;
        const int unit = step * s.width + i;
        if (unit >= s.units) return false;  // padding of a ragged last step: zero nibbles under zero scales
        group = unit / s.rt;
        const int tile = cta + (pass * s.slots + slot) * s.grid;
        which = 0;
        local_tile = tile;
        if (args.pair) {
            which = unit % s.rt;
        } else {
            while (which + 1 < args.count && tile >= args.first_tile[which + 1]) which++;
            local_tile = tile - args.first_tile[which];
        }
        return true;
    };
    auto source_row = [&](const RelayoutSegment &segment, int local_tile, int mma_row) {
        if (segment.rope_head_width > 0) {
            const int tiles_per_head = segment.rope_head_width / 16;
            const int head = local_tile / tiles_per_head, th = local_tile % tiles_per_head;
            const int d = mma_row < 8 ? 8 * th + mma_row : segment.rope_head_width / 2 + 8 * th + (mma_row - 8);
            return head * segment.rope_head_width + d;
        }
        return local_tile * 16 + mma_row;
    };
    const int units = present * s.width;
    for (int index = threadIdx.x; index < units * 64; index += blockDim.x) {
        const int unit_in_stage = index >> 6, half = (index >> 5) & 1, lane = index & 31;
        const int g = lane >> 2, j = lane & 3;
        int group = 0, which = 0, local_tile = 0;
        uint4 value = make_uint4(0, 0, 0, 0);
        if (locate(unit_in_stage, group, which, local_tile)) {
            const RelayoutSegment &segment = args.segment[which];
            const int row = source_row(segment, local_tile, g + 8 * half);
            value = *reinterpret_cast<const uint4 *>(segment.qweight + static_cast<size_t>(row) * (args.k >> 3) + group * 16 + j * 4);
        }
        weights_out[index] = value;
    }
    for (int index = threadIdx.x; index < units * 8; index += blockDim.x) {
        const int unit_in_stage = index >> 3, g = index & 7;
        int group = 0, which = 0, local_tile = 0;
        uint32_t value = 0;
        if (locate(unit_in_stage, group, which, local_tile)) {
            const RelayoutSegment &segment = args.segment[which];
            const uint32_t low = segment.scales[static_cast<size_t>(source_row(segment, local_tile, g)) * groups + group];
            const uint32_t high = segment.scales[static_cast<size_t>(source_row(segment, local_tile, g + 8)) * groups + group];
            value = low | (high << 16);
        }
        scales_out[index] = value;
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
__device__ __forceinline__ void mma_f16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                              uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Two nibbles of `word` (bits 0..3 and 16..19) -> fp16x2 (q - 8, q' - 8), exactly: the nibble lands in the low
// mantissa bits of 1024.0 (0x6400), 1032 is subtracted.
__device__ __forceinline__ uint32_t nibbles_low(uint32_t word) {
    uint32_t biased, out;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(biased) : "r"(word), "n"(0x000F000F), "n"(0x64006400));
    asm("sub.f16x2 %0, %1, %2;" : "=r"(out) : "r"(biased), "r"(0x64086408u));
    return out;
}
// The nibbles at bits 4..7 and 20..23: 1024 + 16 q, times 1/16, minus 72 (one fused multiply-add, exact).
__device__ __forceinline__ uint32_t nibbles_high(uint32_t word) {
    uint32_t biased, out;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(biased) : "r"(word), "n"(0x00F000F0), "n"(0x64006400));
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(out) : "r"(biased), "r"(0x2C002C00u), "r"(0xD480D480u));
    return out;
}

// bf16 values (already rounded) as an fp16 pair: exact for magnitudes in [2^-14, 65504]; the activations of a
// decoder layer (normalised rows, attention outputs, SiLU products) live there.
__device__ __forceinline__ uint32_t half_pair(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&h);
}

__device__ __forceinline__ uint32_t load_acquire(const unsigned int *address) {
    uint32_t value;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(value) : "l"(address) : "memory");
    return value;
}

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 512;" ::: "memory"); }
__device__ __forceinline__ void team_barrier(int barrier_id) { asm volatile("bar.sync %0, 128;" ::"r"(barrier_id) : "memory"); }

// All CTAs of the (cooperative, co-resident) grid meet here; only the consumer warps take part.  `target` counts
// the arrivals expected so far.  A wait that does not complete within the spin limit sets the error flag and lets
// the CTA go on (its results are then garbage, the host sees the flag); once the flag is up nobody waits any more.
__device__ __noinline__ void grid_barrier(unsigned int *counter, unsigned int &target, int *error_flag, unsigned int spin_limit) {
    consumer_sync();
    if (threadIdx.x == 0) {
        target += gridDim.x;
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");  // covers the CTA's writes before the barrier above
        unsigned int spins = 0;
        while (load_acquire(counter) < target) {
            if (++spins > spin_limit) {
                atomicExch(error_flag, 2);
                break;
            }
            if ((spins & 63u) == 0 && *reinterpret_cast<volatile int *>(error_flag) != 0) break;
        }
    }
    consumer_sync();
}

// ---- mbarrier / bulk copy (shared-space addresses)
__device__ __forceinline__ void mbarrier_init(uint32_t address, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(address), "r"(count) : "memory");
}
__device__ __forceinline__ void mbarrier_arrive(uint32_t address) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(address) : "memory");
}
__device__ __forceinline__ void mbarrier_arrive_expect(uint32_t address, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(address), "r"(bytes) : "memory");
}
// One attempt at waiting for the phase of the given parity: the thread is suspended by the hardware until the
// phase completes or about `MBARRIER_SUSPEND_NS` have passed, so a waiting warp issues almost nothing.
constexpr uint32_t MBARRIER_SUSPEND_NS = 20000;
__device__ __forceinline__ bool mbarrier_test(uint32_t address, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(address), "r"(parity), "r"(MBARRIER_SUSPEND_NS)
        : "memory");
    return done != 0;
}
// global -> this CTA's shared memory, completion counted in bytes on `barrier`
__device__ __forceinline__ void bulk_load(uint32_t destination, const void *source, uint32_t bytes, uint32_t barrier) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(destination),
                 "l"(__cvta_generic_to_global(source)), "r"(bytes), "r"(barrier)
                 : "memory");
}
__device__ __forceinline__ void prefetch_l2(const void *address, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(__cvta_generic_to_global(address)), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t shared_load_acquire(uint32_t address) {
    uint32_t value;
    asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(value) : "r"(address) : "memory");
    return value;
}
__device__ __forceinline__ void shared_store_release(uint32_t address, uint32_t value) {
    asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(address), "r"(value) : "memory");
}
// Shared-memory loads by shared-space address (kept in program order behind the waits that make their data valid).
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


// ------------------------------------------------------------------------------------------ the CTA's view of a matrix

struct PhaseInfo {
    int tiles_here;       // 16-row tiles of this CTA (tile = cta + i * grid)
    int passes;           // rounds of `slots` tiles
    int slots, width, steps, units, rt, groups;
    uint32_t cta_offset;  // bytes from the matrix's stream to this CTA's share
    int streamed;         // the activations ride the ring (o, down)
};

struct StackArgs {
    const StackLayer *layers;
    int layer_count;
    StackShape shape;
    StackBuffers buffers;
    LaneTable lanes_meta;
    int lanes, lanes_per_stream, max_splits;
    int stages, stage_bytes, prefetch_stages, debug_flags;
    int steps_per_stage;                 // consecutive steps of a pass that travel as one ring stage (1 or 2)
    int slice_slots, slice_bytes;        // ring of activation slices (o, down) inside the scratch area
    uint32_t scratch_bytes;
    const StackTp *tp;  // device copy of the exchange description, or nullptr (single GPU)
    int tp_size;
};

__device__ __forceinline__ const uint8_t *layer_stream(const StackLayer &layer, int phase) {
    return phase == 0 ? layer.qkv : (phase == 1 ? layer.o : (phase == 2 ? layer.gate_up : layer.down));
}

__device__ __forceinline__ int stage_present(const PhaseInfo &pi, int pass) {
    const int left = pi.tiles_here - pass * pi.slots;
    return left < pi.slots ? left : pi.slots;
}

// ------------------------------------------------------------------------------------------ producers
// Three single threads (lane 0 of warps 16, 17, 18) walk the CTA's stage sequence - for every layer the four
// matrices, for every matrix its passes and steps - each on its own: one requests the weights of a stage, one the
// activation slice of the stages of o and down (once the grid barrier in front of the step has opened), one asks
// L2 for stages further ahead.  A stage's slot is free when the consumer warps have released its previous use
// (the `empty` barrier); its `full` barrier completes with two arrivals plus the bytes of the copies.

struct RingAddresses {
    uint32_t ring, full, empty;                       // weight stages (shared-space addresses)
    uint32_t slices, slice_full, slice_empty;         // activation slices of the o and down steps
    uint32_t open_word, issued_word;
};

struct RingPosition {
    uint32_t slot, parity;  // parity of the `empty` phase that frees the slot for the next use
};
__device__ __forceinline__ void ring_advance(RingPosition &position, uint32_t stages) {
    if (++position.slot == stages) {
        position.slot = 0;
        position.parity ^= 1u;
    }
}
__device__ __forceinline__ void ring_skip(RingPosition &position, uint32_t count, uint32_t stages) {
    const uint32_t to = position.slot + count;
    position.parity ^= (to / stages) & 1u;
    position.slot = to % stages;
}
// false: gave up (the error flag is set, or was set by somebody else)
__device__ __forceinline__ bool wait_slot_free(uint32_t empty_address, const RingPosition &position, int *error_flag) {
    unsigned int spins = 0;
    while (!mbarrier_test(empty_address + position.slot * 8, position.parity)) {
        if (++spins > PIPE_SPIN_LIMIT) {
            atomicExch(error_flag, 3);
            return false;
        }
        if ((spins & 255u) == 0 && *reinterpret_cast<volatile int *>(error_flag) != 0) return false;
    }
    return true;
}
// After giving up: let the copies that are still in flight land before the CTA's shared memory goes away.
__device__ __forceinline__ void linger() {
    for (int i = 0; i < 64; i++) __nanosleep(1000);
}

__device__ __noinline__ void produce_weights(const StackArgs &a, const PhaseInfo *info, const RingAddresses &ring) {
    int *error_flag = a.buffers.error_flag;
    RingPosition position{0u, 1u};
    uint32_t issued = 0;
    for (int layer = 0; layer < a.layer_count; layer++) {
        const StackLayer *spec = a.layers + layer;
        for (int phase = 0; phase < 4; phase++) {
            const PhaseInfo pi = info[phase];
            if (pi.passes == 0) continue;
            const uint8_t *source = layer_stream(*spec, phase) + pi.cta_offset;
            for (int pass = 0; pass < pi.passes; pass++) {
                const uint32_t step_bytes = static_cast<uint32_t>(stage_present(pi, pass) * pi.width * UNIT_TOTAL);
                for (int step = 0; step < pi.steps; step += a.steps_per_stage) {
                    const int count = pi.steps - step < a.steps_per_stage ? pi.steps - step : a.steps_per_stage;
                    const uint32_t bytes = step_bytes * static_cast<uint32_t>(count);
                    if (!wait_slot_free(ring.empty, position, error_flag)) return linger();
                    const uint32_t full = ring.full + position.slot * 8;
                    if ((a.debug_flags & 4) && issued >= static_cast<uint32_t>(a.stages)) {
                        mbarrier_arrive(full);  // timing probe: the consumers work on what the slot already holds
                    } else {
                        mbarrier_arrive_expect(full, bytes);
                        bulk_load(ring.ring + position.slot * static_cast<uint32_t>(a.stage_bytes), source, bytes, full);
                    }
                    source += bytes;
                    ring_advance(position, static_cast<uint32_t>(a.stages));
                    if (a.debug_flags & 4) issued++;
                    if (a.prefetch_stages > 0) asm volatile("st.volatile.shared::cta.u32 [%0], %1;" ::"r"(ring.issued_word), "r"(++issued) : "memory");
                }
            }
        }
    }
}

__device__ __noinline__ void produce_activations(const StackArgs &a, const PhaseInfo *info, const RingAddresses &ring, int staged) {
    int *error_flag = a.buffers.error_flag;
    RingPosition position{0u, 1u};  // in the ring of slices: only the stages of o and down count
    const uint32_t slice_group_bytes = static_cast<uint32_t>(staged) * 256u;
    for (int layer = 0; layer < a.layer_count; layer++) {
        for (int phase = 1; phase < 4; phase += 2) {
            const PhaseInfo pi = info[phase];
            if (pi.passes == 0) continue;
            // the slices were written by other CTAs with ordinary stores before the grid barrier counted here; the
            // scratch area they land in is free once this CTA's consumers have passed that barrier, too
            const uint32_t needed = static_cast<uint32_t>(layer * BARRIERS_PER_LAYER + (phase == 1 ? 2 : 4));
            unsigned int spins = 0;
            while (shared_load_acquire(ring.open_word) < needed) {
                if (++spins > OPEN_SPIN_LIMIT) {
                    atomicExch(error_flag, 3);
                    return linger();
                }
                if ((spins & 255u) == 0 && *reinterpret_cast<volatile int *>(error_flag) != 0) return linger();
                __nanosleep(20);
            }
            asm volatile("fence.proxy.async;" ::: "memory");  // ... and the copy engine reads them
            const uint8_t *base = reinterpret_cast<const uint8_t *>(phase == 1 ? a.buffers.attention_out : a.buffers.activation);
            const int groups_per_stage = pi.width * a.steps_per_stage;
            for (int pass = 0; pass < pi.passes; pass++) {
                for (int first_group = 0; first_group < pi.steps * pi.width; first_group += groups_per_stage) {
                    if (!wait_slot_free(ring.slice_empty, position, error_flag)) return linger();
                    int groups = pi.groups - first_group;
                    if (groups > groups_per_stage) groups = groups_per_stage;
                    const uint32_t full = ring.slice_full + position.slot * 8;
                    if (groups > 0) {
                        const uint32_t bytes = static_cast<uint32_t>(groups) * slice_group_bytes;
                        mbarrier_arrive_expect(full, bytes);
                        bulk_load(ring.slices + position.slot * static_cast<uint32_t>(a.slice_bytes), base + static_cast<size_t>(first_group) * slice_group_bytes,
                                  bytes, full);
                    } else {
                        mbarrier_arrive(full);  // a stage of padding only
                    }
                    ring_advance(position, static_cast<uint32_t>(a.slice_slots));
                }
            }
        }
    }
}

// Keeps `prefetch_stages` stages beyond the last requested one on their way into L2.
__device__ __noinline__ void produce_prefetches(const StackArgs &a, const PhaseInfo *info, const RingAddresses &ring) {
    int *error_flag = a.buffers.error_flag;
    uint32_t index = 0;
    for (int layer = 0; layer < a.layer_count; layer++) {
        const StackLayer *spec = a.layers + layer;
        for (int phase = 0; phase < 4; phase++) {
            const PhaseInfo pi = info[phase];
            if (pi.passes == 0) continue;
            const uint8_t *source = layer_stream(*spec, phase) + pi.cta_offset;
            for (int pass = 0; pass < pi.passes; pass++) {
                const uint32_t step_bytes = static_cast<uint32_t>(stage_present(pi, pass) * pi.width * UNIT_TOTAL);
                for (int step = 0; step < pi.steps; step += a.steps_per_stage, index++) {
                    const int count = pi.steps - step < a.steps_per_stage ? pi.steps - step : a.steps_per_stage;
                    const uint32_t bytes = step_bytes * static_cast<uint32_t>(count);
                    unsigned int spins = 0;
                    uint32_t issued;
                    while (true) {
                        asm volatile("ld.volatile.shared::cta.u32 %0, [%1];" : "=r"(issued) : "r"(ring.issued_word) : "memory");
                        if (index < issued + static_cast<uint32_t>(a.prefetch_stages)) break;
                        if (++spins > OPEN_SPIN_LIMIT || ((spins & 255u) == 0 && *reinterpret_cast<volatile int *>(error_flag) != 0)) return;
                        __nanosleep(100);
                    }
                    if (index >= issued + static_cast<uint32_t>(a.stages)) prefetch_l2(source, bytes);  // nearer stages are being loaded already
                    source += bytes;
                }
            }
        }
    }
}

// Consumer side of the ring: waits (bounded) until stage `slot` holds its data.
__device__ __forceinline__ void wait_stage(uint32_t full_address, uint32_t parity, int *error_flag) {
    unsigned int spins = 0;
    while (!mbarrier_test(full_address, parity)) {
        if (++spins > PIPE_SPIN_LIMIT) {
            atomicExch(error_flag, 3);
            break;
        }
        if ((spins & 255u) == 0 && *reinterpret_cast<volatile int *>(error_flag) != 0) break;
    }
}

// ------------------------------------------------------------------------------------------ activation staging

// Chunk c (8 consecutive columns) of lane m -> the fragment slot of thread (g = m, j) for word w, with
// group = c / 16, j = (c / 4) % 4, w = c % 4: uint4 index ((group * 4 + w) * staged + m) * 4 + j, holding the fp16
// pairs (v0,v4) (v1,v5) (v2,v6) (v3,v7) - the B operands of the MMAs that consume nibble pairs (0,4) (1,5) and
// (2,6) (3,7) of the matching weight word.
__device__ __forceinline__ int fragment_index(int chunk, int m, int staged) {
    const int group = chunk >> 4, j = (chunk >> 2) & 3, word = chunk & 3;
    return ((group * 4 + word) * staged + m) * 4 + j;
}
// Position (in 16-bit elements) of column `column` of lane m in a fragment-ordered buffer.
__device__ __forceinline__ size_t fragment_element(int column, int m, int staged) {
    const int e = column & 7;
    return static_cast<size_t>(fragment_index(column >> 3, m, staged)) * 8 + (e & 3) * 2 + (e >> 2);
}

// rms_norm_bf16.comp.template:49-72 of every staged lane, straight into fragment order (each CTA repeats it:
// 8 KB per lane from L2).  A thread owns chunk t (and t + 512 when CHUNKS = 2) of each lane, four lanes at a time:
// one pass over registers for the sums of squares, one block-wide exchange, then normalise, round and permute.
// Two f32 values rounded to bf16 (nearest even, as the shaders' f32_to_bf16 for every finite value) and carried on
// as the fp16 pair the tensor cores read: exact, a bf16 of this range fits fp16.
__device__ __forceinline__ uint32_t bf16_rounded_half_pair(float lo, float hi) {
    uint32_t packed, halves;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(packed) : "f"(hi), "f"(lo));
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(halves) : "f"(bf16_hi(packed)), "f"(bf16_lo(packed)));
    return halves;
}

template <int CHUNKS>  // chunks per thread and lane: width <= CHUNKS * 8 * CONSUMER_THREADS
__device__ __noinline__ void stage_normalised(uint4 *fragments, float *partial, const uint16_t *x, const uint16_t *weight, int width,
                                                 int staged, float eps, float offset) {
    const int per_lane = width >> 3, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint4 *source = reinterpret_cast<const uint4 *>(x);
    uint4 scale_words[CHUNKS];
#pragma unroll
    for (int c = 0; c < CHUNKS; c++) {
        const int chunk = threadIdx.x + c * CONSUMER_THREADS;
        scale_words[c] = chunk < per_lane ? __ldg(reinterpret_cast<const uint4 *>(weight) + chunk) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll 1
    for (int m0 = 0; m0 < staged; m0 += 4) {
        uint4 raw[4][CHUNKS];
#pragma unroll
        for (int mm = 0; mm < 4; mm++)
#pragma unroll
            for (int c = 0; c < CHUNKS; c++) {
                const int chunk = threadIdx.x + c * CONSUMER_THREADS;
                // lanes beyond the batch read the last lane again (their results are not stored)
                const int m = m0 + mm < staged ? m0 + mm : staged - 1;
                raw[mm][c] = __ldcg(source + static_cast<size_t>(m) * per_lane + (chunk < per_lane ? chunk : 0));
            }
        float sums[4];
#pragma unroll
        for (int mm = 0; mm < 4; mm++) {
            float sum = 0.0f;
#pragma unroll
            for (int c = 0; c < CHUNKS; c++) {
                if (CHUNKS > 1 && threadIdx.x + c * CONSUMER_THREADS >= per_lane) continue;
                const uint32_t words[4] = {raw[mm][c].x, raw[mm][c].y, raw[mm][c].z, raw[mm][c].w};
#pragma unroll
                for (int w = 0; w < 4; w++) {
                    const float lo = bf16_lo(words[w]), hi = bf16_hi(words[w]);
                    sum = fmaf(lo, lo, sum);
                    sum = fmaf(hi, hi, sum);
                }
            }
            sums[mm] = (CHUNKS > 1 || static_cast<int>(threadIdx.x) < per_lane) ? sum : 0.0f;
        }
        // the four sums cross the warp together: after two exchanges a thread holds the sum of lane 2 * bit0 + bit1
        {
            const bool odd = lane & 1;
            const float keep0 = odd ? sums[2] : sums[0], keep1 = odd ? sums[3] : sums[1];
            const float send0 = odd ? sums[0] : sums[2], send1 = odd ? sums[1] : sums[3];
            const float a0 = keep0 + __shfl_xor_sync(0xffffffffu, send0, 1), a1 = keep1 + __shfl_xor_sync(0xffffffffu, send1, 1);
            const bool upper = lane & 2;
            float sum = (upper ? a1 : a0) + __shfl_xor_sync(0xffffffffu, upper ? a0 : a1, 2);
            sum += __shfl_xor_sync(0xffffffffu, sum, 4);
            sum += __shfl_xor_sync(0xffffffffu, sum, 8);
            sum += __shfl_xor_sync(0xffffffffu, sum, 16);
            if (lane < 4) partial[(2 * (lane & 1) + (lane >> 1)) * CONSUMER_WARPS + warp] = sum;
        }
        consumer_sync();
        // every warp adds up the 16 partials of the four lanes: lanes 8k .. 8k+7 of the warp take lane m0 + k
        float total = partial[(lane >> 3) * CONSUMER_WARPS + (lane & 7) * 2] + partial[(lane >> 3) * CONSUMER_WARPS + (lane & 7) * 2 + 1];
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
                const int chunk = threadIdx.x + c * CONSUMER_THREADS;
                if (chunk < per_lane && m0 + mm < staged) {
                    const uint32_t in[4] = {raw[mm][c].x, raw[mm][c].y, raw[mm][c].z, raw[mm][c].w};
                    const uint32_t sc[4] = {scale_words[c].x, scale_words[c].y, scale_words[c].z, scale_words[c].w};
                    float v[8];
#pragma unroll
                    for (int w = 0; w < 4; w++) {
                        v[2 * w] = bf16_lo(in[w]) * inv_rms * (bf16_lo(sc[w]) + offset);
                        v[2 * w + 1] = bf16_hi(in[w]) * inv_rms * (bf16_hi(sc[w]) + offset);
                    }
                    fragments[fragment_index(chunk, m0 + mm, staged)] =
                        make_uint4(bf16_rounded_half_pair(v[0], v[4]), bf16_rounded_half_pair(v[1], v[5]), bf16_rounded_half_pair(v[2], v[6]),
                                   bf16_rounded_half_pair(v[3], v[7]));
                }
            }
        }
        if (m0 + 4 < staged) consumer_sync();  // `partial` is rewritten for the next four lanes
    }
    consumer_sync();
}

// ------------------------------------------------------------------------------------------ attention
// A team of four warps serves one context split (64 tokens) of one kv head for the Q = QL * GROUP <= 16 query
// vectors of QL consecutive lanes of a stream (append_gqa_attention_bf16.comp.template:217-339: f32 scores of
// bf16 q.k, f32 softmax, f32 p.v); warp w of the team takes tokens 16w .. 16w + 15 of the split.  Scores and p.v
// run on the tensor cores: q rows are the A operand of S = Q K^T, K rows the B operand (both read with 16-byte
// loads; the head dimension is permuted identically on both sides); the probabilities are re-used from the
// accumulator registers as the A operand of O = P V, split into a bf16 high and low part (p = hi + lo to 2^-17),
// and V is the B operand, its token pairs assembled with byte permutes.  The warps agree on the split's row
// maxima through shared memory, add up their partial outputs there (HALF head dims per pass), and the team writes
// one partial (unnormalised output, maximum, sum) per query to the scratch.  The team that completes a kv head's
// last split merges all of them (log-sum-exp) and writes the head's outputs, fp16 in fragment order, where the o
// projection's activation slices are copied from.

template <int HD>
__host__ __device__ constexpr size_t attention_team_bytes() {
    return (4 * 16 * ((HD < 64 ? HD : 64) + 4) + 2 * 4 * 16 + 4) * sizeof(float);  // partial outputs [warp][row][HALF + 4], maxima and sums [warp][row], one flag
}

struct AttentionJob {  // what every attention item of a launch shares
    const uint16_t *q;
    float *scratch;
    uint16_t *out_fragments;
    unsigned int *arrivals;
    int lanes, lanes_per_stream, q_heads, kv_heads, max_splits, group_slots, staged;
    float scale;
};
// The scratch of a layer's attention step: every (lane, q head, split) partial is HD floats of unnormalised output in
// `values` [lane][q head][split][HD] (16-byte aligned rows) and (maximum, sum) in `stats` [lane][q head][split][2]
// behind all the values - together the (HD + 2) floats per partial the scratch is sized for.
__device__ __forceinline__ float *attention_stats(float *scratch, int lanes, int q_heads, int max_splits, int head_width) {
    return scratch + static_cast<size_t>(lanes) * q_heads * max_splits * head_width;
}

// Log-sum-exp merge of up to 32 partials of one (lane, q head) row by one warp: lane s of the warp weighs partial s,
// every lane owns HD / 32 consecutive output dims, and the weighted rows are summed in order, the loads of eight or
// sixteen partials in flight at a time.  `values` points at the lane's dims of the first partial (rows of HD floats),
// `stats` at its (maximum, sum).  Leaves the block's maximum, its sum and the lane's unnormalised dims.
constexpr int MERGE_BLOCK = 32;
template <int HD>
__device__ __forceinline__ void attention_merge_block(const float *__restrict__ values, const float2 *__restrict__ stats, int count, float &maximum,
                                                      float &denominator, float (&acc)[HD / 32]) {
    constexpr int VEC = HD / 32;
    static_assert(VEC == 1 || VEC == 2 || VEC == 4, "a lane owns one, two or four output dims");
    constexpr int CHUNK = VEC == 4 ? 8 : 16;  // rows in flight at a time; a divisor of the block, whose weights sit in the warp's lanes
    static_assert(MERGE_BLOCK % CHUNK == 0, "rounds of the merge must not straddle a block");
    const int lane_id = threadIdx.x & 31;
    const int last = count - 1;
    // Rows beyond the last partial are read as the last one again and weigh nothing, so no load is predicated.
    float part[CHUNK][VEC];
    auto fetch = [&](int first) {
#pragma unroll
        for (int u = 0; u < CHUNK; u++) {
            const float *source = values + static_cast<size_t>(first + u < last ? first + u : last) * HD;
            if (VEC == 4) {
                const float4 raw = __ldcg(reinterpret_cast<const float4 *>(source));
                part[u][0] = raw.x, part[u][VEC > 1 ? 1 : 0] = raw.y, part[u][VEC > 2 ? 2 : 0] = raw.z, part[u][VEC > 3 ? 3 : 0] = raw.w;
            } else if (VEC == 2) {
                const float2 raw = __ldcg(reinterpret_cast<const float2 *>(source));
                part[u][0] = raw.x, part[u][VEC > 1 ? 1 : 0] = raw.y;
            } else {
                part[u][0] = __ldcg(source);
            }
        }
    };
#pragma unroll
    for (int v = 0; v < VEC; v++) acc[v] = 0.0f;
    // the statistics and the first rows are requested together
    const float2 pair = __ldcg(stats + (lane_id < last ? lane_id : last));
    fetch(0);
    maximum = warp_max(lane_id < count ? pair.x : -3.4028234663852886e38f);
    const float weight = lane_id < count ? expf(pair.x - maximum) : 0.0f;
    denominator = warp_sum(lane_id < count ? pair.y * weight : 0.0f);
#pragma unroll 1
    for (int s = 0; s < count; s += CHUNK) {
        if (s != 0) fetch(s);
#pragma unroll
        for (int u = 0; u < CHUNK; u++) {
            const float w = __shfl_sync(0xffffffffu, weight, s + u);  // 0 in the lanes beyond the last partial
#pragma unroll
            for (int v = 0; v < VEC; v++) acc[v] += part[u][v] * w;
        }
    }
}

// How many 64-token splits the partials of a query lane's rows cover: those of the newest lane of its group of QL
// lanes (a team writes every row of its group for every split of the group; rows of older lanes are masked there).
__device__ __forceinline__ int attention_group_splits(const AttentionJob &job, const uint32_t *ticks, uint32_t capacity, int query_lane, int ql) {
    const int stream = query_lane / job.lanes_per_stream, first = ((query_lane % job.lanes_per_stream) / ql) * ql;
    uint32_t tick = 0;
    for (int i = first; i < first + ql && i < job.lanes_per_stream; i++) {
        const uint32_t other = ticks[stream * job.lanes_per_stream + i];
        if (other > tick) tick = other;
    }
    const uint32_t tokens = tick + 1u < capacity ? tick + 1u : capacity;
    const int splits = static_cast<int>((tokens + 63u) / 64u);
    return splits < job.max_splits ? splits : job.max_splits;
}

// The splits of one lane's own attended window.
__device__ __forceinline__ int attention_own_splits(const AttentionJob &job, uint32_t capacity, uint32_t tick) {
    const uint32_t tokens = tick + 1u < capacity ? tick + 1u : capacity;
    const int splits = static_cast<int>((tokens + 63u) / 64u);
    return splits < job.max_splits ? splits : job.max_splits;
}

// The scratch behind the split partials: per row and range of MERGE_BLOCK splits one merged partial, laid out like
// the split partials (values, then statistics).  Used by rows of more than MERGE_BLOCK splits.
__device__ __forceinline__ float *attention_range_values(const AttentionJob &job, int head_width) {
    return job.scratch + static_cast<size_t>(job.lanes) * job.q_heads * job.max_splits * (head_width + 2);
}
__device__ __forceinline__ int attention_ranges(int max_splits) { return (max_splits + MERGE_BLOCK - 1) / MERGE_BLOCK; }

// A row of at most MERGE_BLOCK splits: merged and written out as fp16 in fragment order by one warp.
template <int HD>
__device__ __noinline__ void attention_merge_row(const AttentionJob &job, int splits, int query_lane, int head) {
    constexpr int VEC = HD / 32;
    const int lane_id = threadIdx.x & 31;
    const size_t row = (static_cast<size_t>(query_lane) * job.q_heads + head) * job.max_splits;
    float maximum, denominator, acc[VEC];
    attention_merge_block<HD>(job.scratch + row * HD + lane_id * VEC,
                              reinterpret_cast<const float2 *>(attention_stats(job.scratch, job.lanes, job.q_heads, job.max_splits, HD)) + row, splits, maximum,
                              denominator, acc);
#pragma unroll
    for (int v = 0; v < VEC; v++) {
        const float rounded = round_bf16(denominator == 0.0f ? 0.0f : acc[v] / denominator);
        job.out_fragments[fragment_element(head * HD + lane_id * VEC + v, query_lane, job.staged)] = __half_as_ushort(__float2half_rn(rounded));
    }
}

// Longer rows, first level: one range of MERGE_BLOCK splits of a row into one partial.
template <int HD>
__device__ __noinline__ void attention_merge_range(const AttentionJob &job, int splits, int query_lane, int head, int range) {
    constexpr int VEC = HD / 32;
    const int lane_id = threadIdx.x & 31;
    const size_t row = static_cast<size_t>(query_lane) * job.q_heads + head;
    const size_t first = row * job.max_splits + static_cast<size_t>(range) * MERGE_BLOCK;
    const int count = splits - range * MERGE_BLOCK < MERGE_BLOCK ? splits - range * MERGE_BLOCK : MERGE_BLOCK;
    float maximum, denominator, acc[VEC];
    attention_merge_block<HD>(job.scratch + first * HD + lane_id * VEC,
                              reinterpret_cast<const float2 *>(attention_stats(job.scratch, job.lanes, job.q_heads, job.max_splits, HD)) + first, count, maximum,
                              denominator, acc);
    const int ranges = attention_ranges(job.max_splits);
    float *values = attention_range_values(job, HD);
    float *out = values + (row * ranges + range) * HD + lane_id * VEC;
#pragma unroll
    for (int v = 0; v < VEC; v++) out[v] = acc[v];
    if (lane_id == 0) {
        float2 *statistics = reinterpret_cast<float2 *>(values + static_cast<size_t>(job.lanes) * job.q_heads * ranges * HD) + row * ranges + range;
        *statistics = make_float2(maximum, denominator);
    }
}

// Second level: the row's range partials merged and written out.
template <int HD>
__device__ __noinline__ void attention_merge_ranges(const AttentionJob &job, int splits, int query_lane, int head) {
    constexpr int VEC = HD / 32;
    const int lane_id = threadIdx.x & 31;
    const size_t row = static_cast<size_t>(query_lane) * job.q_heads + head;
    const int ranges = attention_ranges(job.max_splits), count = (splits + MERGE_BLOCK - 1) / MERGE_BLOCK;
    const float *values = attention_range_values(job, HD);
    float maximum, denominator, acc[VEC];
    attention_merge_block<HD>(values + row * ranges * HD + lane_id * VEC,
                              reinterpret_cast<const float2 *>(values + static_cast<size_t>(job.lanes) * job.q_heads * ranges * HD) + row * ranges, count, maximum,
                              denominator, acc);
#pragma unroll
    for (int v = 0; v < VEC; v++) {
        const float rounded = round_bf16(denominator == 0.0f ? 0.0f : acc[v] / denominator);
        job.out_fragments[fragment_element(head * HD + lane_id * VEC + v, query_lane, job.staged)] = __half_as_ushort(__float2half_rn(rounded));
    }
}

// Loads through L2 that stay where they are written (the compiler may not sink them towards their use).
__device__ __forceinline__ uint4 load16_now(const void *address) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(address) : "memory");
    return v;
}
__device__ __forceinline__ uint2 load8_now(const void *address) {
    uint2 v;
    asm volatile("ld.global.cg.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(address) : "memory");
    return v;
}

template <int HD>
__device__ __noinline__ size_t attention_row_base(const KvLayer &kv, int slot, uint32_t ring_base, int token) {
    uint32_t ring = ring_base + static_cast<uint32_t>(token);
    if (ring >= kv.capacity) ring -= kv.capacity;
    const int page = static_cast<int>(ring / kv.page_tokens), within = static_cast<int>(ring % kv.page_tokens);
    const int physical = kv.block_table[static_cast<size_t>(slot) * kv.pages_per_slot + page];
    return static_cast<size_t>(physical) * 2 * kv.kv_heads * kv.page_tokens * HD + static_cast<size_t>(within) * HD;
}

constexpr int ATTENTION_MERGE_LIST = 63;
// Per-CTA copies of what every layer needs again: the lanes' ticks and stream slots, and for each team the KV rows
// of its first work item (the block table is shared by all layers, so the rows of a (split, lane group) are the
// same in every layer's pool).
struct AttentionCache {
    AttentionJob job;
    uint32_t tick[8];
    int32_t slot[8];
    int32_t item[4];          // the work item whose rows `row_base` holds, or -1
    int32_t rows[4];          // how many tokens that item has
    int32_t merge_count;      // (kv head, lane group) pairs whose last split this CTA's teams completed in this layer ...
    int32_t merge_list[ATTENTION_MERGE_LIST];  // ... and which: kv_head * group_slots + group_slot
    uint32_t row_base[4][64]; // offset (in rows of HD elements) of token t's K row of kv head 0 in a layer's pool
    StackLayer layer[2];      // the current layer's description (layer & 1) and the next one's, copied ahead of their use
};

template <int HD, int GROUP, int QL>
__device__ __noinline__ void attention_team_item(AttentionCache &cache, const KvLayer &kv_shared, int item, uint8_t *scratch_area,
                                                    unsigned long long *stamps) {
    constexpr int Q = QL * GROUP;
    // the launch's and the layer's descriptions by value: behind a reference every field would be read again after
    // each of the ordered loads below
    const KvLayer kv = kv_shared;
    const AttentionJob job = cache.job;
    const uint16_t *__restrict__ q = job.q;
    float *__restrict__ scratch = job.scratch;
    const int lanes = job.lanes, lanes_per_stream = job.lanes_per_stream, q_heads = job.q_heads, max_splits = job.max_splits;
    const int group_slots = job.group_slots;
    const float scale = job.scale;
    const int team = static_cast<int>(threadIdx.x >> 7), team_warp = static_cast<int>(threadIdx.x >> 5) & 3, barrier_id = 2 + team;
    float *team_smem = reinterpret_cast<float *>(scratch_area + static_cast<size_t>(team) * attention_team_bytes<HD>());
    const int kv_head = item % job.kv_heads, split = (item / job.kv_heads) % max_splits, group_slot = (item / job.kv_heads) / max_splits;
    unsigned int *__restrict__ arrivals = job.arrivals;
    auto mark = [&](int index) {
        if (stamps != nullptr) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            stamps[index] = now;
        }
    };
    constexpr int QW = HD / 32;                    // 16-byte pieces of a q / k row per thread
    constexpr int HALF = HD < 64 ? HD : 64;        // head dims handled per output pass
    constexpr int DPT = HALF / 8;                  // of which one thread column owns this many
    static_assert(Q <= 16 && HD % 32 == 0, "attention team shape");
    const int lane = threadIdx.x & 31, g = lane >> 2, j = lane & 3;
    constexpr int PITCH = HALF + 4;                       // row pitch of the partial outputs (bank spread)
    float *partial_out = team_smem;                       // [4][16][PITCH]
    float *team_max = team_smem + 4 * 16 * PITCH;         // [4][16]
    float *team_sum = team_max + 4 * 16;                  // [4][16]
    unsigned int *team_flag = reinterpret_cast<unsigned int *>(team_sum + 4 * 16);
    const int groups_per_stream = (lanes_per_stream + QL - 1) / QL;
    const int stream_index = group_slot / groups_per_stream, group_index = group_slot % groups_per_stream;
    const int lane0 = stream_index * lanes_per_stream + group_index * QL;
    if (lane0 >= lanes) return;
    const int slot = cache.slot[lane0];
    if (slot < 0) return;
    const uint32_t capacity = kv.capacity;

    uint32_t newest = 0, tick_row[2] = {0xffffffffu, 0xffffffffu};
#pragma unroll
    for (int i = 0; i < QL; i++) {
        const bool valid = lane0 + i < lanes && group_index * QL + i < lanes_per_stream;
        const uint32_t tick = valid ? cache.tick[lane0 + i] : 0xffffffffu;
        if (valid && tick > newest) newest = tick;
        if (g < Q && g / GROUP == i) tick_row[0] = tick;
        if (g + 8 < Q && (g + 8) / GROUP == i) tick_row[1] = tick;
    }
    const uint32_t tokens = newest + 1u < capacity ? newest + 1u : capacity;  // attended window of the newest lane
    const uint32_t first_tick = newest + 1u - tokens;
    const uint32_t begin = static_cast<uint32_t>(split) * 64u;
    if (begin >= tokens) return;  // the whole team leaves: nobody waits at the team barrier
    mark(20);
    int expected_splits = static_cast<int>((tokens + 63u) / 64u);
    if (expected_splits > max_splits) expected_splits = max_splits;
    const int count = static_cast<int>(tokens - begin < 64u ? tokens - begin : 64u);
    const int token0 = 16 * team_warp;  // this warp's tokens of the split
    // element offset of token t's K (or V) row of this kv head: from the team's cached rows, or through the block table
    const size_t half_page = static_cast<size_t>(kv.kv_heads) * kv.page_tokens * HD;
    const bool cached = cache.item[team] == item;
    const uint32_t ring_base = (first_tick + begin) % capacity;
    // Row numbers (units of HD elements, kv head 0) of the K rows this thread reads (tokens g and g + 8 of the warp's
    // sixteen) and of its V rows (tokens 2j, 2j + 1, 2j + 8, 2j + 9).  Without cached rows every thread walks the
    // block table for one token and the warp passes the rows round: one dependent load instead of six in a row.
    uint32_t k_row[2], v_row[4];
    if (cached) {
#pragma unroll
        for (int nt = 0; nt < 2; nt++) k_row[nt] = cache.row_base[team][(token0 + nt * 8 + g) & 63];
#pragma unroll
        for (int t = 0; t < 4; t++) v_row[t] = cache.row_base[team][(token0 + 2 * j + (t & 1) + 8 * (t >> 1)) & 63];
    } else {
        const int token = token0 + (lane & 15);
        const uint32_t mine = token < count ? static_cast<uint32_t>(attention_row_base<HD>(kv, slot, ring_base, token) / HD) : 0u;
#pragma unroll
        for (int nt = 0; nt < 2; nt++) k_row[nt] = __shfl_sync(0xffffffffu, mine, nt * 8 + g);
#pragma unroll
        for (int t = 0; t < 4; t++) v_row[t] = __shfl_sync(0xffffffffu, mine, 2 * j + (t & 1) + 8 * (t >> 1));
    }
    const size_t head_offset = static_cast<size_t>(kv_head) * kv.page_tokens * HD;

    // ---- S = Q K^T for 16 tokens.  The team's Q query rows go to shared memory with asynchronous copies (they
    // would otherwise hold 32 registers per thread while the K and V rows are in flight); a row is kept as HD / 32
    // pieces of 64 bytes, thread column j reading 16 bytes of each - K rows are read from memory the same way, so
    // the head dimension is permuted identically on both sides of the product.
    constexpr uint32_t Q_PITCH = HD * 2 + 64;  // bytes; 16-byte reads of a quarter warp fall into distinct banks
    const uint32_t q_shared = static_cast<uint32_t>(__cvta_generic_to_shared(partial_out));  // free until the first output pass
    {
        const int team_thread = team_warp * 32 + lane;
        for (int piece = team_thread; piece < 16 * QW * 4; piece += 128) {
            const int row = piece / (QW * 4), part = piece % (QW * 4);
            const int query_lane = lane0 + row / GROUP;
            const bool valid = row < Q && query_lane < lanes && group_index * QL + row / GROUP < lanes_per_stream;
            const uint32_t destination = q_shared + static_cast<uint32_t>(row) * Q_PITCH + static_cast<uint32_t>(part) * 16u;
            if (valid) {
                const uint16_t *source = q + (static_cast<size_t>(query_lane) * q_heads + kv_head * GROUP + row % GROUP) * HD + part * 8;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(destination), "l"(source) : "memory");
            } else {
                asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(destination), "r"(0u) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    // K rows of tokens g and g + 8, V rows of tokens 2j, 2j+1, 2j+8, 2j+9 of this warp: all requested before the
    // arithmetic (the V rows of the first output pass now, those of the second when the q registers are free)
    uint4 kf[2][QW];
#pragma unroll
    for (int nt = 0; nt < 2; nt++) {
        const int token = token0 + nt * 8 + g;
        if (token < count) {
            const uint16_t *krow = kv.pool + static_cast<size_t>(k_row[nt]) * HD + head_offset + j * 8;
#pragma unroll
            for (int w = 0; w < QW; w++) kf[nt][w] = load16_now(krow + w * 32);
        } else {
#pragma unroll
            for (int w = 0; w < QW; w++) kf[nt][w] = make_uint4(0, 0, 0, 0);
        }
    }
    size_t v_offset[4];
#pragma unroll
    for (int t = 0; t < 4; t++) {
        const int token = token0 + 2 * j + (t & 1) + 8 * (t >> 1);
        v_offset[t] = token < count ? static_cast<size_t>(v_row[t]) * HD + half_page + head_offset : static_cast<size_t>(-1);
    }
    uint32_t v[HD / HALF][4][DPT / 2];
    auto load_values = [&](int pass) {
#pragma unroll
        for (int t = 0; t < 4; t++) {
            if (v_offset[t] != static_cast<size_t>(-1)) {
                const uint16_t *vrow = kv.pool + v_offset[t] + pass * HALF + DPT * g;
                if (DPT == 8) {
                    const uint4 raw = load16_now(vrow);
                    v[pass][t][0] = raw.x;
                    v[pass][t][1] = raw.y;
                    v[pass][t][DPT / 2 - 2] = raw.z;
                    v[pass][t][DPT / 2 - 1] = raw.w;
                } else {
                    const uint2 raw = load8_now(vrow);
                    v[pass][t][0] = raw.x;
                    v[pass][t][DPT / 2 - 1] = raw.y;
                }
            } else {
#pragma unroll
                for (int w = 0; w < DPT / 2; w++) v[pass][t][w] = 0u;
            }
        }
    };
    load_values(0);
    asm volatile("cp.async.wait_all;" ::: "memory");
    team_barrier(barrier_id);  // the query rows are in shared memory
    float s[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; nt++) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
#pragma unroll
    for (int w = 0; w < QW; w++) {
        const uint32_t at = q_shared + static_cast<uint32_t>(g) * Q_PITCH + static_cast<uint32_t>(w) * 64u + static_cast<uint32_t>(j) * 16u;
        const uint4 q0 = shared_load16<0>(at), q1 = shared_load16<8 * Q_PITCH>(at);
#pragma unroll
        for (int nt = 0; nt < 2; nt++) {
            mma_bf16_16816(s[nt], q0.x, q1.x, q0.y, q1.y, kf[nt][w].x, kf[nt][w].y);
            mma_bf16_16816(s[nt], q0.z, q1.z, q0.w, q1.w, kf[nt][w].z, kf[nt][w].w);
        }
    }
    if (HD / HALF > 1) load_values(HD / HALF - 1);
    mark(21);

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
    mark(22);
    // probabilities as the A fragment of this warp's 16 tokens: high and low bf16 parts
    uint32_t ph[4], pl[4];
#pragma unroll
    for (int f = 0; f < 4; f++) {
        const float first = s[f >> 1][2 * (f & 1)], second = s[f >> 1][2 * (f & 1) + 1];
        ph[f] = pack_bf16(first, second);
        pl[f] = pack_bf16(first - bf16_lo(ph[f]), second - bf16_hi(ph[f]));
    }

    // ---- O = P V over the warp's tokens, HALF head dims per pass; thread column g owns dims DPT*g .. DPT*g+DPT-1
    float *mine = partial_out + static_cast<size_t>(team_warp) * 16 * PITCH;
#pragma unroll
    for (int pass = 0; pass < HD / HALF; pass++) {
        float o[DPT][4];
#pragma unroll
        for (int i = 0; i < DPT; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
#pragma unroll
        for (int i = 0; i < DPT; i++) {
            const uint32_t selector = (i & 1) ? 0x7632u : 0x5410u;
            const uint32_t b0 = __byte_perm(v[pass][0][i >> 1], v[pass][1][i >> 1], selector), b1 = __byte_perm(v[pass][2][i >> 1], v[pass][3][i >> 1], selector);
            mma_bf16_16816(o[i], ph[0], ph[1], ph[2], ph[3], b0, b1);
            mma_bf16_16816(o[i], pl[0], pl[1], pl[2], pl[3], b0, b1);
        }
        // accumulator column 2j (+1) of output tile i is head dim DPT * (2j (+1)) + i of the pass
#pragma unroll
        for (int r = 0; r < 2; r++)
#pragma unroll
            for (int half = 0; half < 2; half++)
#pragma unroll
                for (int i = 0; i < DPT; i += 4)
                    *reinterpret_cast<float4 *>(mine + (g + 8 * r) * PITCH + DPT * (2 * j + half) + i) =
                        make_float4(o[i][2 * r + half], o[i + 1][2 * r + half], o[i + 2][2 * r + half], o[i + 3][2 * r + half]);
        team_barrier(barrier_id);
        // the four partial outputs add up; warp w writes dims [w * HALF / 4, (w + 1) * HALF / 4) of the pass for every
        // row, four dims per thread and round
        constexpr int QUADS = HALF / 16;
#pragma unroll
        for (int round = 0; round < (16 * QUADS + 31) / 32; round++) {
            const int task = round * 32 + lane, row = task / QUADS, d = team_warp * (HALF / 4) + (task % QUADS) * 4;
            const int query_lane = lane0 + row / GROUP;  // rows beyond Q are padding
            if (row < Q && query_lane < lanes && group_index * QL + row / GROUP < lanes_per_stream) {
                const float *in = partial_out + row * PITCH + d;
                const float4 p0 = *reinterpret_cast<const float4 *>(in), p1 = *reinterpret_cast<const float4 *>(in + 16 * PITCH),
                             p2 = *reinterpret_cast<const float4 *>(in + 32 * PITCH), p3 = *reinterpret_cast<const float4 *>(in + 48 * PITCH);
                const size_t partial = (static_cast<size_t>(query_lane) * q_heads + kv_head * GROUP + row % GROUP) * max_splits + split;
                *reinterpret_cast<float4 *>(scratch + partial * HD + pass * HALF + d) =
                    make_float4(p0.x + p1.x + p2.x + p3.x, p0.y + p1.y + p2.y + p3.y, p0.z + p1.z + p2.z + p3.z, p0.w + p1.w + p2.w + p3.w);
            }
        }
        if (pass == 0 && team_warp == 0 && lane < Q) {
            const int row = lane, query_lane = lane0 + row / GROUP;
            if (query_lane < lanes && group_index * QL + row / GROUP < lanes_per_stream) {
                const size_t partial = (static_cast<size_t>(query_lane) * q_heads + kv_head * GROUP + row % GROUP) * max_splits + split;
                *reinterpret_cast<float2 *>(attention_stats(scratch, lanes, q_heads, max_splits, HD) + partial * 2) = make_float2(
                    fmaxf(fmaxf(fmaxf(team_max[row], team_max[16 + row]), fmaxf(team_max[32 + row], team_max[48 + row])), -3.4028234663852886e38f),
                    team_sum[row] + team_sum[16 + row] + team_sum[32 + row] + team_sum[48 + row]);
            }
        }
        if (pass + 1 < HD / HALF) team_barrier(barrier_id);  // the partial outputs are rewritten by the next pass
    }
    // ---- the team that completes the kv head's last split merges the splits of its queries; groups of more than
    // MERGE_BLOCK splits are merged in two levels by the whole grid after the items
    mark(23);
    if (expected_splits > MERGE_BLOCK) {
        team_barrier(barrier_id);  // the team's shared arrays are free for its next item
        return;
    }
    __threadfence();
    team_barrier(barrier_id);
    unsigned int *arrival = arrivals + kv_head * group_slots + group_slot;
    if (team_warp == 0 && lane == 0) *team_flag = atomicAdd(arrival, 1u);
    team_barrier(barrier_id);
    const bool last = *team_flag == static_cast<unsigned int>(expected_splits - 1);
    mark(24);
    if (last) {
        // all splits of this kv head and lane group are in the scratch: the CTA merges them after its items (one row
        // per warp); a CTA with more such heads than its list holds merges the rest right here
        team_barrier(barrier_id);  // everybody has read the flag
        if (team_warp == 0 && lane == 0) {
            __threadfence();
            *arrival = 0u;  // for the next layer (several grid barriers away)
            const int request = atomicAdd(&cache.merge_count, 1);
            if (request < ATTENTION_MERGE_LIST) cache.merge_list[request] = kv_head * group_slots + group_slot;
            *team_flag = static_cast<unsigned int>(request);
        }
        team_barrier(barrier_id);
        if (*team_flag >= static_cast<unsigned int>(ATTENTION_MERGE_LIST)) {
            __threadfence();
            for (int row = team_warp; row < Q; row += 4) {
                const int query_lane = lane0 + row / GROUP;
                if (query_lane < lanes && group_index * QL + row / GROUP < lanes_per_stream)
                    attention_merge_row<HD>(cache.job, attention_own_splits(cache.job, capacity, cache.tick[query_lane]), query_lane,
                                            kv_head * GROUP + row % GROUP);
            }
        }
    }
    team_barrier(barrier_id);  // the team's shared arrays are free for its next item
    mark(25);
}

template <int GROUP>
struct AttentionTeam {
    static constexpr int QL = GROUP >= 8 ? 2 : (GROUP >= 4 ? 4 : (16 / GROUP > 8 ? 8 : 16 / GROUP));
};

// ------------------------------------------------------------------------------------------ matrix blocks

// One 16x128 block at `weights` (this thread's 16 bytes of rows g and, 512 bytes on, g + 8) against the staged
// activations of its group: eight MMAs over exact fp16 (q - 8) operands in two accumulation chains.
struct UnitOperands {
    uint4 low, high;  // this thread's 32 nibbles of rows g and g + 8
    uint4 b[4];       // its B fragments of the block's group
    uint32_t scales;  // bf16 scale of row g | row g + 8
};
__device__ __forceinline__ void unit_load(UnitOperands &u, uint32_t weights, uint32_t scales, uint32_t x, uint32_t word_stride) {
    u.b[0] = shared_load16<0>(x);
    u.b[1] = shared_load16<0>(x + word_stride);
    u.b[2] = shared_load16<0>(x + 2 * word_stride);
    u.b[3] = shared_load16<0>(x + 3 * word_stride);
    u.low = shared_load16<0>(weights);
    u.high = shared_load16<512>(weights);
    u.scales = shared_load4(scales);
}
// Word `WORD` of the block: two MMAs into two of the block's four accumulation chains.
template <int WORD>
__device__ __forceinline__ void unit_word(const UnitOperands &u, float (&chains)[4][4]) {
    const uint32_t wa = WORD == 0 ? u.low.x : (WORD == 1 ? u.low.y : (WORD == 2 ? u.low.z : u.low.w));
    const uint32_t wb = WORD == 0 ? u.high.x : (WORD == 1 ? u.high.y : (WORD == 2 ? u.high.z : u.high.w));
    const uint4 &b = u.b[WORD];
    mma_f16_16816(chains[2 * (WORD & 1)], nibbles_low(wa), nibbles_low(wb), nibbles_high(wa), nibbles_high(wb), b.x, b.y);
    const uint32_t upper_a = wa >> 8, upper_b = wb >> 8;
    mma_f16_16816(chains[2 * (WORD & 1) + 1], nibbles_low(upper_a), nibbles_low(upper_b), nibbles_high(upper_a), nibbles_high(upper_b), b.z, b.w);
}
__device__ __forceinline__ void unit_finish(const UnitOperands &u, const float (&chains)[4][4], float (&acc)[4]) {
    const float sa = __uint_as_float(u.scales << 16), sb = __uint_as_float(u.scales & 0xffff0000u);
    acc[0] = fmaf(sa, (chains[0][0] + chains[1][0]) + (chains[2][0] + chains[3][0]), acc[0]);
    acc[1] = fmaf(sa, (chains[0][1] + chains[1][1]) + (chains[2][1] + chains[3][1]), acc[1]);
    acc[2] = fmaf(sb, (chains[0][2] + chains[1][2]) + (chains[2][2] + chains[3][2]), acc[2]);
    acc[3] = fmaf(sb, (chains[0][3] + chains[1][3]) + (chains[2][3] + chains[3][3]), acc[3]);
}
// One 16x128 block against the staged activations of its group: eight MMAs over exact fp16 (q - 8) operands in
// four accumulation chains; the group scale multiplies the block's f32 product.
__device__ __forceinline__ void unit_single(const UnitOperands &u, float (&acc)[4]) {
    float chains[4][4] = {};
    unit_word<0>(u, chains);
    unit_word<1>(u, chains);
    unit_word<2>(u, chains);
    unit_word<3>(u, chains);
    unit_finish(u, chains, acc);
}
// Two blocks at once, their MMAs interleaved (eight independent chains).
__device__ __forceinline__ void unit_pair(const UnitOperands &u, const UnitOperands &v, float (&acc)[4]) {
    float cu[4][4] = {}, cv[4][4] = {};
    unit_word<0>(u, cu);
    unit_word<0>(v, cv);
    unit_word<1>(u, cu);
    unit_word<1>(v, cv);
    unit_word<2>(u, cu);
    unit_word<2>(v, cv);
    unit_word<3>(u, cu);
    unit_word<3>(v, cv);
    unit_finish(u, cu, acc);
    unit_finish(v, cv, acc);
}

// The steps of one pass as a warp sees them, in a function of its own so that the loop's registers are allotted
// apart from the long-lived state of the kernel body.  For every stage of the pass: wait until it has landed,
// multiply this warp's block (if it has one in this stage) and release the stage.  `x` is the shared-space address
// of the thread's B fragments of the first step - relative to the stage for activation slices that ride the ring,
// absolute (moving on by x_step per step) for the normalised rows.
struct PassResult {
    float acc[4];
    uint32_t slot, parity, slice_slot, slice_parity;
    uint32_t payload[4];  // what the epilogue needs from global memory (the residual values), requested before the steps
};
struct PassRing {  // where the stages are and where this warp stands in them
    uint32_t ring, full, empty, stages, stage_bytes;
    uint32_t slices, slice_full, slice_empty, slice_slots, slice_bytes;
};
template <bool X_IN_SLICE, int PER_STAGE>
__device__ __noinline__ PassResult consume_pass(const PassRing ring, uint32_t slot, uint32_t parity, uint32_t slice_slot, uint32_t slice_parity,
                                                int steps, int active_steps, uint32_t step_bytes, uint32_t weight_offset,
                                                uint32_t scale_offset, uint32_t x, uint32_t x_step, uint32_t word_stride,
                                                int *error_flag, const uint16_t *payload, uint32_t payload_stride, int payload_rounds) {
    constexpr bool x_in_slice = X_IN_SLICE;
    constexpr int steps_per_stage = PER_STAGE;
    constexpr bool handshake = true;
    uint32_t residual[4];
#pragma unroll
    for (int round = 0; round < 4; round++) residual[round] = round < payload_rounds ? __ldcg(payload + static_cast<size_t>(round) * payload_stride) : 0;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    const int lane = threadIdx.x & 31;
    for (int step = 0; step < steps; step += steps_per_stage) {
        const uint32_t stage_address = ring.ring + slot * ring.stage_bytes;
        const uint32_t slice_address = ring.slices + slice_slot * ring.slice_bytes;
        if (handshake) {
            wait_stage(ring.full + slot * 8, parity, error_flag);
            if (x_in_slice) wait_stage(ring.slice_full + slice_slot * 8, slice_parity, error_flag);
        }
        int here = active_steps - step;  // this warp's blocks in the stage
        if (here > steps_per_stage) here = steps_per_stage;
        if (here > 0) {
            const uint32_t x_first = x_in_slice ? slice_address + x : x;
            UnitOperands u;
            unit_load(u, stage_address + weight_offset, stage_address + scale_offset, x_first, word_stride);
            unit_single(u, acc);
            if (PER_STAGE == 2 && here == 2) {
                unit_load(u, stage_address + step_bytes + weight_offset, stage_address + step_bytes + scale_offset, x_first + x_step, word_stride);
                unit_single(u, acc);
            }
            if (!x_in_slice) x += static_cast<uint32_t>(here) * x_step;
        }
        __syncwarp();
        if (lane == 0 && handshake) {
            mbarrier_arrive(ring.empty + slot * 8);
            if (x_in_slice) mbarrier_arrive(ring.slice_empty + slice_slot * 8);
        }
        if (++slot == ring.stages) {
            slot = 0;
            parity ^= 1u;
        }
        if (x_in_slice && ++slice_slot == ring.slice_slots) {
            slice_slot = 0;
            slice_parity ^= 1u;
        }
    }
    PassResult result;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        result.acc[i] = acc[i];
        result.payload[i] = residual[i];
    }
    result.slot = slot;
    result.parity = parity;
    result.slice_slot = slice_slot;
    result.slice_parity = slice_parity;
    return result;
}

// The gate/up step when a stage holds two steps of two blocks per tile slot (gate and up of one group of K each):
// the slot's two warps take one step each and multiply BOTH its blocks - gate and up rows against the same
// activations, read once - with the sixteen MMAs interleaved in eight accumulation chains.  Returns the warp's partial
// sums of the gate rows (acc) and of the up rows (second).
struct PairResult {
    float acc[4], second[4];
    uint32_t slot, parity;
};
struct PairOperands {
    uint4 low_a, high_a, low_b, high_b;  // this thread's nibbles of rows g and g + 8: gate block, up block
    uint4 b[4];                          // its B fragments of the group
    uint32_t scales_a, scales_b;
};
template <int WORD>
__device__ __forceinline__ void pair_word(const PairOperands &p, float (&ca)[4][4], float (&cb)[4][4]) {
    const uint4 &b = p.b[WORD];
    const uint32_t wa = WORD == 0 ? p.low_a.x : (WORD == 1 ? p.low_a.y : (WORD == 2 ? p.low_a.z : p.low_a.w));
    const uint32_t wb = WORD == 0 ? p.high_a.x : (WORD == 1 ? p.high_a.y : (WORD == 2 ? p.high_a.z : p.high_a.w));
    const uint32_t va = WORD == 0 ? p.low_b.x : (WORD == 1 ? p.low_b.y : (WORD == 2 ? p.low_b.z : p.low_b.w));
    const uint32_t vb = WORD == 0 ? p.high_b.x : (WORD == 1 ? p.high_b.y : (WORD == 2 ? p.high_b.z : p.high_b.w));
    mma_f16_16816(ca[2 * (WORD & 1)], nibbles_low(wa), nibbles_low(wb), nibbles_high(wa), nibbles_high(wb), b.x, b.y);
    mma_f16_16816(cb[2 * (WORD & 1)], nibbles_low(va), nibbles_low(vb), nibbles_high(va), nibbles_high(vb), b.x, b.y);
    const uint32_t upper_wa = wa >> 8, upper_wb = wb >> 8, upper_va = va >> 8, upper_vb = vb >> 8;
    mma_f16_16816(ca[2 * (WORD & 1) + 1], nibbles_low(upper_wa), nibbles_low(upper_wb), nibbles_high(upper_wa), nibbles_high(upper_wb), b.z, b.w);
    mma_f16_16816(cb[2 * (WORD & 1) + 1], nibbles_low(upper_va), nibbles_low(upper_vb), nibbles_high(upper_va), nibbles_high(upper_vb), b.z, b.w);
}
__device__ __forceinline__ void pair_finish(uint32_t scales, const float (&chains)[4][4], float (&acc)[4]) {
    const float sa = __uint_as_float(scales << 16), sb = __uint_as_float(scales & 0xffff0000u);
    acc[0] = fmaf(sa, (chains[0][0] + chains[1][0]) + (chains[2][0] + chains[3][0]), acc[0]);
    acc[1] = fmaf(sa, (chains[0][1] + chains[1][1]) + (chains[2][1] + chains[3][1]), acc[1]);
    acc[2] = fmaf(sb, (chains[0][2] + chains[1][2]) + (chains[2][2] + chains[3][2]), acc[2]);
    acc[3] = fmaf(sb, (chains[0][3] + chains[1][3]) + (chains[2][3] + chains[3][3]), acc[3]);
}
// `first_block`: byte offset of the gate block of the warp's slot inside a step; `first_scales`: of its scale row;
// `mine`: which of the stage's two steps this warp takes; `x`: its B fragments of that step's group in the first stage.
__device__ __noinline__ PairResult consume_pass_pairs(const PassRing ring, uint32_t slot, uint32_t parity, int steps, bool active, int mine, uint32_t step_bytes,
                                                      uint32_t first_block, uint32_t first_scales, uint32_t x, uint32_t x_stage_step, uint32_t word_stride,
                                                      int *error_flag) {
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f}, second[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    const int lane = threadIdx.x & 31;
    for (int step = 0; step < steps; step += 2) {
        const uint32_t stage_address = ring.ring + slot * ring.stage_bytes;
        wait_stage(ring.full + slot * 8, parity, error_flag);
        if (active && step + mine < steps) {
            const uint32_t base = stage_address + static_cast<uint32_t>(mine) * step_bytes;
            PairOperands p;
            p.b[0] = shared_load16<0>(x);
            p.b[1] = shared_load16<0>(x + word_stride);
            p.b[2] = shared_load16<0>(x + 2 * word_stride);
            p.b[3] = shared_load16<0>(x + 3 * word_stride);
            p.low_a = shared_load16<0>(base + first_block);
            p.high_a = shared_load16<512>(base + first_block);
            p.low_b = shared_load16<UNIT_BYTES>(base + first_block);
            p.high_b = shared_load16<UNIT_BYTES + 512>(base + first_block);
            p.scales_a = shared_load4(base + first_scales);
            p.scales_b = shared_load4(base + first_scales + UNIT_SCALE_BYTES);
            float ca[4][4] = {}, cb[4][4] = {};
            pair_word<0>(p, ca, cb);
            pair_word<1>(p, ca, cb);
            pair_word<2>(p, ca, cb);
            pair_word<3>(p, ca, cb);
            pair_finish(p.scales_a, ca, acc);
            pair_finish(p.scales_b, cb, second);
            x += x_stage_step;
        }
        __syncwarp();
        if (lane == 0) mbarrier_arrive(ring.empty + slot * 8);
        if (++slot == ring.stages) {
            slot = 0;
            parity ^= 1u;
        }
    }
    PairResult result;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        result.acc[i] = acc[i];
        result.second[i] = second[i];
    }
    result.slot = slot;
    result.parity = parity;
    return result;
}

// ------------------------------------------------------------------------------------------ the kernel

// EXCHANGE: the tensor-parallel form (o and down leave partial sums that are exchanged between the ranks).
template <int HD, int GROUP, bool EXCHANGE>
__global__ void __launch_bounds__(STACK_THREADS, 1) decode_stack_kernel(const StackArgs a) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    if (a.buffers.timing != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        a.buffers.timing[16] = now;
    }
    constexpr int QL = AttentionTeam<GROUP>::QL;
    const StackShape &shape = a.shape;
    const int lanes = a.lanes, staged = lanes < 8 ? lanes : 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, j = lane & 3;

    // shared memory: scratch (fragments / attention teams) | reduce [2][16][16][8] f32 | norm partials | phase table |
    // barriers | ring
    uint4 *fragments = reinterpret_cast<uint4 *>(smem_raw);
    float *reduce = reinterpret_cast<float *>(smem_raw + a.scratch_bytes);
    float *norm_partial = reduce + 2 * CONSUMER_WARPS * 128;
    uint32_t *rope_rows = reinterpret_cast<uint32_t *>(norm_partial + 4 * CONSUMER_WARPS);  // [8 lanes][HD / 2] rotary factors of the lanes' positions
    AttentionCache *attention_cache = reinterpret_cast<AttentionCache *>(rope_rows + 8 * (HD >> 1));
    PhaseInfo *info = reinterpret_cast<PhaseInfo *>(attention_cache + 1);
    uint64_t *barriers = reinterpret_cast<uint64_t *>(info + 4);
    uint32_t *open_word = reinterpret_cast<uint32_t *>(barriers + 4 * MAX_STAGES);  // [0] grid barriers passed, [1] stages requested
    uint8_t *ring_base = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(open_word + 4) + 127) & ~static_cast<uintptr_t>(127));
    RingAddresses ring;
    ring.ring = static_cast<uint32_t>(__cvta_generic_to_shared(ring_base));
    ring.full = static_cast<uint32_t>(__cvta_generic_to_shared(barriers));
    ring.empty = ring.full + MAX_STAGES * 8;
    ring.slices = static_cast<uint32_t>(__cvta_generic_to_shared(smem_raw));  // the slices share the scratch area with the fragments
    ring.slice_full = ring.empty + MAX_STAGES * 8;
    ring.slice_empty = ring.slice_full + MAX_STAGES * 8;
    ring.open_word = static_cast<uint32_t>(__cvta_generic_to_shared(open_word));
    ring.issued_word = ring.open_word + 4;

    const int q_width = shape.q_heads * HD, kv_width = shape.kv_heads * HD;
    const int q_tiles = q_width >> 4, k_tiles = kv_width >> 4;
    if (threadIdx.x == 0) {
        const int grid = static_cast<int>(gridDim.x), cta = static_cast<int>(blockIdx.x);
        const MatrixSchedule schedules[4] = {stack_schedule((q_width + 2 * kv_width) >> 4, shape.hidden >> 7, 1, grid),
                                             stack_schedule(shape.hidden >> 4, q_width >> 7, 1, grid),
                                             stack_schedule(shape.ffn >> 4, shape.hidden >> 7, 2, grid),
                                             stack_schedule(shape.hidden >> 4, shape.ffn >> 7, 1, grid)};
        for (int p = 0; p < 4; p++) {
            const MatrixSchedule &s = schedules[p];
            PhaseInfo pi;
            pi.tiles_here = stack_cta_tiles(s, cta);
            pi.passes = (pi.tiles_here + s.slots - 1) / s.slots;
            pi.slots = s.slots;
            pi.width = s.width;
            pi.steps = s.steps;
            pi.units = s.units;
            pi.rt = s.rt;
            pi.groups = s.units / s.rt;
            pi.cta_offset = static_cast<uint32_t>(stack_cta_offset(s, cta));
            pi.streamed = (p == 1 || p == 3) ? 1 : 0;
            info[p] = pi;
        }
        for (int s = 0; s < a.stages; s++) {
            mbarrier_init(ring.full + s * 8, 1);                 // the producer's arrival with the byte count
            mbarrier_init(ring.empty + s * 8, CONSUMER_WARPS);  // one arrival per consumer warp
        }
        for (int s = 0; s < a.slice_slots; s++) {
            mbarrier_init(ring.slice_full + s * 8, 1);
            mbarrier_init(ring.slice_empty + s * 8, CONSUMER_WARPS);
        }
        open_word[0] = 0u;
        open_word[1] = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async;" ::: "memory");
    }
    __syncthreads();

    if (warp >= CONSUMER_WARPS) {
        if (lane == 0) {
            if (warp == CONSUMER_WARPS) produce_weights(a, info, ring);
            else if (warp == CONSUMER_WARPS + 1) produce_activations(a, info, ring, staged);
            else if (warp == CONSUMER_WARPS + 2 && a.prefetch_stages > 0) produce_prefetches(a, info, ring);
        }
        return;
    }

    // ------------------------------------------------------------------ consumers
    unsigned int target = a.buffers.barrier_handicap, barriers_passed = 0;
    const unsigned int barrier_spin_limit = a.buffers.barrier_handicap != 0 ? (1u << 12) : BARRIER_SPIN_LIMIT;
    unsigned int *counter = a.buffers.barrier;
    int *error_flag = a.buffers.error_flag;
    uint32_t tag = 0;  // exchanges done so far, earlier launches included
    unsigned long long *inbox_mine = nullptr;
    if constexpr (EXCHANGE) {
        tag = static_cast<uint32_t>(a.tp->counter[a.tp->rank][STACK_TP_WORD_CONSUMED]);
        inbox_mine = reinterpret_cast<unsigned long long *>(a.tp->exchange[a.tp->rank]);
    }
    uint32_t ring_slot = 0, ring_parity = 0, slice_slot = 0, slice_parity = 0;
    int reduce_parity = 0;
    PassRing pass_ring;
    pass_ring.ring = ring.ring;
    pass_ring.full = ring.full;
    pass_ring.empty = ring.empty;
    pass_ring.stages = static_cast<uint32_t>(a.stages);
    pass_ring.stage_bytes = static_cast<uint32_t>(a.stage_bytes);
    pass_ring.slices = ring.slices;
    pass_ring.slice_full = ring.slice_full;
    pass_ring.slice_empty = ring.slice_empty;
    pass_ring.slice_slots = static_cast<uint32_t>(a.slice_slots);
    pass_ring.slice_bytes = static_cast<uint32_t>(a.slice_bytes);

    auto stamp = [&](int layer, int index) {
        if (a.buffers.timing != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            a.buffers.timing[layer * 32 + index] = now;
        }
    };
    auto meet = [&]() {
        grid_barrier(counter, target, error_flag, barrier_spin_limit);
        barriers_passed++;
        if (threadIdx.x == 0) shared_store_release(ring.open_word, barriers_passed);
    };

    // Epilogue roles: thread t finishes output (high = t & 1, lane m = (t >> 1) & 7, row = ((t >> 4) & 7) + 8 * high)
    // of tile slot (t >> 7) + 4 * round, so the rotary partner rows r and r + 8 of a lane sit in neighbouring threads.
    const int epilogue_m = (threadIdx.x >> 1) & 7, epilogue_row = ((threadIdx.x >> 4) & 7) + 8 * (threadIdx.x & 1);
    const int epilogue_slot = threadIdx.x >> 7;
    const bool epilogue_lane = epilogue_m < lanes;
    // per-lane constants of the epilogue: position, rotary table row, and the lane's KV row inside a page (the
    // block table is shared by all layers)
    uint32_t lane_position = 0;
    size_t kv_token_base = 0;
    bool kv_writable = false;
    if (epilogue_lane) {
        lane_position = a.lanes_meta.position[epilogue_m];
        const KvLayer &kv0 = a.layers[0].kv;
        const int slot = a.lanes_meta.slot[epilogue_m];
        if (slot >= 0 && kv0.capacity != 0) {
            const uint32_t ring_token = lane_position % kv0.capacity;
            const int physical = kv0.block_table[static_cast<size_t>(slot) * kv0.pages_per_slot + ring_token / kv0.page_tokens];
            kv_token_base = static_cast<size_t>(physical) * 2 * kv0.kv_heads * kv0.page_tokens * HD + static_cast<size_t>(ring_token % kv0.page_tokens) * HD;
            kv_writable = true;
        }
    }
    for (int index = threadIdx.x; index < staged * (HD >> 1); index += CONSUMER_THREADS) {
        const int m = index / (HD >> 1);
        rope_rows[index] = __ldg(shape.rope_table + static_cast<size_t>(a.lanes_meta.position[m] % shape.rope_positions) * (HD >> 1) + (index - m * (HD >> 1)));
    }
    constexpr int LAYER_WORDS = static_cast<int>(sizeof(StackLayer) / sizeof(uint32_t));
    static_assert(sizeof(StackLayer) % sizeof(uint32_t) == 0, "layer descriptions are copied word by word");
    if (threadIdx.x >= 32 && threadIdx.x < 32 + LAYER_WORDS)
        reinterpret_cast<uint32_t *>(&attention_cache->layer[0])[threadIdx.x - 32] = reinterpret_cast<const uint32_t *>(a.layers)[threadIdx.x - 32];
    if (threadIdx.x < 8) {
        attention_cache->tick[threadIdx.x] = static_cast<int>(threadIdx.x) < lanes ? a.lanes_meta.position[threadIdx.x] : 0u;
        attention_cache->slot[threadIdx.x] = static_cast<int>(threadIdx.x) < lanes ? a.lanes_meta.slot[threadIdx.x] : -1;
    }
    consumer_sync();
    {
        // the KV rows of each team's first attention item, looked up once for all layers
        const int streams = lanes / a.lanes_per_stream;
        const int groups_per_stream = (a.lanes_per_stream + QL - 1) / QL;
        const int group_slots = streams * groups_per_stream;
        const int total = shape.kv_heads * a.max_splits * group_slots;
        const int team = warp >> 2, team_thread = threadIdx.x & 127;
        const int item = static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) * team;
        int cached_item = -1, cached_rows = 0;
        if (item < total) {
            const int rest = item / shape.kv_heads, split = rest % a.max_splits, group_slot = rest / a.max_splits;
            const int lane0 = (group_slot / groups_per_stream) * a.lanes_per_stream + (group_slot % groups_per_stream) * QL;
            const KvLayer &kv0 = a.layers[0].kv;
            const int slot = lane0 < lanes ? attention_cache->slot[lane0] : -1;
            if (slot >= 0 && kv0.capacity != 0) {
                uint32_t newest = 0;
                for (int i = 0; i < QL; i++)
                    if (lane0 + i < lanes && (group_slot % groups_per_stream) * QL + i < a.lanes_per_stream && attention_cache->tick[lane0 + i] > newest)
                        newest = attention_cache->tick[lane0 + i];
                const uint32_t tokens = newest + 1u < kv0.capacity ? newest + 1u : kv0.capacity;
                const uint32_t begin = static_cast<uint32_t>(split) * 64u;
                if (begin < tokens) {
                    const uint32_t ring_base = (newest + 1u - tokens + begin) % kv0.capacity;
                    if (team_thread < 64 && begin + team_thread < tokens)
                        attention_cache->row_base[team][team_thread] = static_cast<uint32_t>(attention_row_base<HD>(kv0, slot, ring_base, team_thread) / HD);
                    cached_item = item;
                    cached_rows = static_cast<int>(tokens - begin < 64u ? tokens - begin : 64u);
                }
            }
        }
        if (threadIdx.x == 0) {
            attention_cache->merge_count = 0;
            AttentionJob job;
            job.q = a.buffers.q;
            job.scratch = a.buffers.attention_scratch;
            job.out_fragments = a.buffers.attention_out;
            job.arrivals = a.buffers.barrier + ARRIVAL_WORDS_OFFSET;
            job.lanes = lanes;
            job.lanes_per_stream = a.lanes_per_stream;
            job.q_heads = shape.q_heads;
            job.kv_heads = shape.kv_heads;
            job.max_splits = a.max_splits;
            job.group_slots = group_slots;
            job.staged = staged;
            job.scale = shape.attention_scale;
            attention_cache->job = job;
        }
        if (team_thread == 0) {
            attention_cache->item[team] = cached_item;
            attention_cache->rows[team] = cached_rows;
        }
    }
    consumer_sync();
    // gate/up in pairs (consume_pass_pairs): when a stage is two steps of (gate, up) blocks per tile slot and the scratch
    // has room for the up rows' partial sums behind the normalised rows
    const size_t pair_reduce_offset = static_cast<size_t>(staged) * shape.hidden * 2;
    // (two copies, alternating like the main array, when the step takes several passes)
    const int pair_copies = info[2].passes > 1 ? 2 : 1;
    const bool pairs_enabled = info[2].rt == 2 && info[2].width == 2 && a.steps_per_stage == 2 && !(a.debug_flags & 1) &&
                               pair_reduce_offset + pair_copies * CONSUMER_WARPS * 128 * sizeof(float) <= a.scratch_bytes;
    float *reduce_second = reinterpret_cast<float *>(smem_raw + pair_reduce_offset);
    const int ge = g < staged ? g : 0;  // lanes beyond the batch recompute lane 0; their results are dropped
    const uint32_t fragment_lane = static_cast<uint32_t>(__cvta_generic_to_shared(fragments)) + static_cast<uint32_t>(ge * 4 + j) * 16u;
    const uint32_t word_stride = static_cast<uint32_t>(staged) * 4 * sizeof(uint4);  // between the four words of a group
    const uint32_t group_stride = 4 * word_stride;
    const int grid = static_cast<int>(gridDim.x);

    for (int layer = 0; layer < a.layer_count; layer++) {
        const StackLayer *spec = &attention_cache->layer[layer & 1];
        const KvLayer kv = spec->kv;
        // the next layer's description: into the other copy (last read before the previous layer's final barrier)
        if (threadIdx.x >= 32 && threadIdx.x < 32 + LAYER_WORDS && layer + 1 < a.layer_count)
            reinterpret_cast<uint32_t *>(&attention_cache->layer[(layer + 1) & 1])[threadIdx.x - 32] =
                reinterpret_cast<const uint32_t *>(a.layers + layer + 1)[threadIdx.x - 32];
        {
            // the K and V rows this CTA's teams will read in this layer's attention step: on their way into L2 now
            const int team = warp >> 2, team_thread = threadIdx.x & 127;
            const int item = attention_cache->item[team];
            if (item >= 0 && team_thread < attention_cache->rows[team] && kv.capacity != 0) {
                const int kv_head = item % shape.kv_heads;
                const size_t half_page = static_cast<size_t>(kv.kv_heads) * kv.page_tokens * HD;
                const uint16_t *row = kv.pool + static_cast<size_t>(attention_cache->row_base[team][team_thread]) * HD + static_cast<size_t>(kv_head) * kv.page_tokens * HD;
#pragma unroll
                for (int line = 0; line < (HD * 2 + 127) / 128; line++) {
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const uint8_t *>(row) + line * 128));
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const uint8_t *>(row + half_page) + line * 128));
                }
            }
        }
        for (int phase = 0; phase < 4; phase++) {
            const PhaseInfo pi = info[phase];
            stamp(layer, 4 * phase);
            // ---- activations of q/k/v and gate/up: normalised rows into fragment order
            if (phase == 0 || phase == 2) {
                const uint16_t *norm_weight = phase == 0 ? spec->input_norm : spec->post_norm;
                if (shape.hidden <= 8 * CONSUMER_THREADS)
                    stage_normalised<1>(fragments, norm_partial, a.buffers.hidden, norm_weight, shape.hidden, staged, shape.eps, shape.norm_offset);
                else
                    stage_normalised<2>(fragments, norm_partial, a.buffers.hidden, norm_weight, shape.hidden, staged, shape.eps, shape.norm_offset);
            }
            stamp(layer, 4 * phase + 1);

            const int slot_of_warp = warp / pi.width, index_in_slot = warp - slot_of_warp * pi.width;
            for (int pass = 0; pass < pi.passes; pass++) {
                const int present = stage_present(pi, pass);
                const bool active = warp < present * pi.width;
                // the epilogue's residual values are requested before the arithmetic: rounds of four tile slots
                const uint16_t *payload_address = a.buffers.hidden;
                int payload_rounds = 0;
                if (epilogue_lane && (phase == 1 || phase == 3) && epilogue_slot < present) {
                    payload_address = a.buffers.hidden + static_cast<size_t>(epilogue_m) * shape.hidden +
                                      (static_cast<size_t>(blockIdx.x) + static_cast<size_t>(pass * pi.slots + epilogue_slot) * grid) * 16 + epilogue_row;
                    payload_rounds = (present - epilogue_slot + 3) / 4;
                }
                // this warp's units of the pass: index_in_slot, + width, ... while below `units`
                int active_steps = 0;
                if (active && index_in_slot < pi.units && !(a.debug_flags & 1)) active_steps = (pi.units - index_in_slot + pi.width - 1) / pi.width;
                const uint32_t lane_fragment = static_cast<uint32_t>(ge * 4 + j) * 16u;
                // B fragments: of the group the warp's first unit belongs to - in the slice of the stage (o, down), or in
                // the normalised rows, moving on by width / rt groups per step
                const uint32_t x_step = static_cast<uint32_t>(pi.width / pi.rt) * group_stride;
                const uint32_t x_start = pi.streamed ? static_cast<uint32_t>(index_in_slot) * group_stride + lane_fragment
                                                     : fragment_lane + static_cast<uint32_t>(index_in_slot / pi.rt) * group_stride;
                const bool pair_mode = phase == 2 && pairs_enabled;
                PassResult done;
                float second_acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                if (pair_mode) {
                    const PairResult pairs = consume_pass_pairs(pass_ring, ring_slot, ring_parity, pi.steps, active, index_in_slot,
                                                                static_cast<uint32_t>(present * pi.width * UNIT_TOTAL),
                                                                static_cast<uint32_t>(slot_of_warp * 2) * UNIT_BYTES + static_cast<uint32_t>(lane) * 16u,
                                                                static_cast<uint32_t>(present * pi.width) * UNIT_BYTES +
                                                                    static_cast<uint32_t>(slot_of_warp * 2) * UNIT_SCALE_BYTES + static_cast<uint32_t>(g) * 4u,
                                                                fragment_lane + static_cast<uint32_t>(index_in_slot) * group_stride, 2 * group_stride, word_stride,
                                                                error_flag);
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        done.acc[i] = pairs.acc[i];
                        second_acc[i] = pairs.second[i];
                        done.payload[i] = 0;
                    }
                    done.slot = pairs.slot;
                    done.parity = pairs.parity;
                    done.slice_slot = slice_slot;
                    done.slice_parity = slice_parity;
                } else {
                    const uint32_t step_bytes = static_cast<uint32_t>(present * pi.width * UNIT_TOTAL);
                    const uint32_t weight_offset = static_cast<uint32_t>(warp) * UNIT_BYTES + static_cast<uint32_t>(lane) * 16u;
                    const uint32_t scale_offset = static_cast<uint32_t>(present * pi.width) * UNIT_BYTES + static_cast<uint32_t>(warp) * UNIT_SCALE_BYTES +
                                                  static_cast<uint32_t>(g) * 4u;
                    const uint32_t payload_stride = static_cast<uint32_t>(4 * grid * 16);
                    if (a.steps_per_stage == 2) {
                        done = pi.streamed ? consume_pass<true, 2>(pass_ring, ring_slot, ring_parity, slice_slot, slice_parity, pi.steps, active_steps, step_bytes,
                                                                   weight_offset, scale_offset, x_start, x_step, word_stride, error_flag, payload_address,
                                                                   payload_stride, payload_rounds)
                                           : consume_pass<false, 2>(pass_ring, ring_slot, ring_parity, slice_slot, slice_parity, pi.steps, active_steps, step_bytes,
                                                                    weight_offset, scale_offset, x_start, x_step, word_stride, error_flag, payload_address,
                                                                    payload_stride, payload_rounds);
                    } else {
                        done = pi.streamed ? consume_pass<true, 1>(pass_ring, ring_slot, ring_parity, slice_slot, slice_parity, pi.steps, active_steps, step_bytes,
                                                                   weight_offset, scale_offset, x_start, x_step, word_stride, error_flag, payload_address,
                                                                   payload_stride, payload_rounds)
                                           : consume_pass<false, 1>(pass_ring, ring_slot, ring_parity, slice_slot, slice_parity, pi.steps, active_steps, step_bytes,
                                                                    weight_offset, scale_offset, x_start, x_step, word_stride, error_flag, payload_address,
                                                                    payload_stride, payload_rounds);
                    }
                }
                ring_slot = done.slot;
                ring_parity = done.parity;
                slice_slot = done.slice_slot;
                slice_parity = done.slice_parity;
                stamp(layer, 26 + phase);
                const float (&acc)[4] = done.acc;
                // ---- the warps' partial sums meet: reduce[parity][warp][row][lane]
                float *mine = reduce + static_cast<size_t>((reduce_parity * CONSUMER_WARPS + warp) * 128);
                *reinterpret_cast<float2 *>(mine + g * 8 + 2 * j) = make_float2(acc[0], acc[1]);
                *reinterpret_cast<float2 *>(mine + (g + 8) * 8 + 2 * j) = make_float2(acc[2], acc[3]);
                if (pair_mode) {
                    float *up = reduce_second + static_cast<size_t>(((pair_copies == 2 ? reduce_parity : 0) * CONSUMER_WARPS + warp) * 128);
                    *reinterpret_cast<float2 *>(up + g * 8 + 2 * j) = make_float2(second_acc[0], second_acc[1]);
                    *reinterpret_cast<float2 *>(up + (g + 8) * 8 + 2 * j) = make_float2(second_acc[2], second_acc[3]);
                }
                consumer_sync();
                const float *sums = reduce + static_cast<size_t>(reduce_parity * CONSUMER_WARPS * 128);
                const float *second_sums = reduce_second + static_cast<size_t>((pair_copies == 2 ? reduce_parity : 0) * CONSUMER_WARPS * 128);
                reduce_parity ^= 1;
#pragma unroll 1
                for (int round = 0; round < 4; round++) {
                    const int slot = epilogue_slot + 4 * round;
                    if (slot >= present) break;  // uniform over the warp
                    const int tile = static_cast<int>(blockIdx.x) + (pass * pi.slots + slot) * grid;
                    const float *src = sums + static_cast<size_t>(slot * pi.width) * 128 + epilogue_row * 8 + epilogue_m;
                    float first = 0.0f, second = 0.0f;
                    if (pair_mode) {
                        // both warps of the slot hold gate sums (here) and up sums (in the second array), of alternate groups
                        const float *up = second_sums + static_cast<size_t>(slot * pi.width) * 128 + epilogue_row * 8 + epilogue_m;
                        first = src[0] + src[128];
                        second = up[0] + up[128];
                    } else if (pi.rt == 2) {
                        for (int w = 0; w < pi.width; w += 2) {
                            first += src[w * 128];
                            second += src[(w + 1) * 128];
                        }
                    } else {
                        for (int w = 0; w < pi.width; w++) first += src[w * 128];
                    }
                    if (phase == 0) {
                        // q / k: rotary_bf16.comp.template:99-109 (non-interleaved, rotary width = head width, five bf16
                        // roundings); k and v go into the lane's KV page (append_gqa_attention_bf16.comp.template:189-215)
                        const float mine_value = round_bf16(first);
                        const float partner = __shfl_xor_sync(0xffffffffu, mine_value, 1);  // the row 8 further (or 8 back)
                        if (epilogue_lane) {
                            const size_t kv_half = static_cast<size_t>(kv.kv_heads) * kv.page_tokens * HD;
                            if (tile < q_tiles + k_tiles) {
                                const bool is_q = tile < q_tiles, high = epilogue_row >= 8;
                                const int local = is_q ? tile : tile - q_tiles;
                                const int head = local / (HD >> 4), d = 8 * (local % (HD >> 4)) + (epilogue_row & 7) + (high ? HD / 2 : 0);
                                const uint32_t rotation = rope_rows[epilogue_m * (HD >> 1) + 8 * (local % (HD >> 4)) + (epilogue_row & 7)];
                                const float cosine = bf16_lo(rotation), sine = bf16_hi(rotation);
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
                    } else if (epilogue_lane) {
                        const int column = tile * 16 + epilogue_row;
                        if (phase == 2) {
                            // silu_multiply_bf16.comp.template:30-52: bf16(silu_bf16(bf16 gate) * bf16 up), kept as fp16 in
                            // fragment order for the down projection
                            const float product = round_bf16(rounded_silu(round_bf16(first)) * round_bf16(second));
                            a.buffers.activation[fragment_element(column, epilogue_m, staged)] = __half_as_ushort(__float2half_rn(product));
                        } else {
                            float total = first;
                            if constexpr (EXCHANGE) {
                                // this rank's share of the sum over K goes to every peer's inbox, value and exchange number in
                                // one 8-byte store; the peers' shares arrive in this rank's inbox the same way
                                const StackTp &tp = *a.tp;
                                const uint32_t number = tag + 1u;
                                const size_t element = (static_cast<size_t>(number & 1u) * STACK_TP_MAX_RANKS * 8 + epilogue_m) * shape.hidden + column;
                                const unsigned long long word = (static_cast<unsigned long long>(number) << 32) | __float_as_uint(first);
                                for (int r = 0; r < tp.size; r++)
                                    if (r != tp.rank)
                                        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(reinterpret_cast<unsigned long long *>(tp.exchange[r]) + element +
                                                                                              static_cast<size_t>(tp.rank) * 8 * shape.hidden),
                                                     "l"(word)
                                                     : "memory");
                                total = 0.0f;
                                unsigned int spins = 0;
                                bool gave_up = false;
                                for (int r = 0; r < tp.size; r++) {  // rank order on every rank: the replicas stay bit-identical
                                    float part = first;
                                    if (r != tp.rank) {
                                        const unsigned long long *source = inbox_mine + element + static_cast<size_t>(r) * 8 * shape.hidden;
                                        unsigned long long got = 0;
                                        while (!gave_up) {
                                            asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(got) : "l"(source) : "memory");
                                            if (static_cast<uint32_t>(got >> 32) == number) break;
                                            if (++spins > STACK_TP_SPIN_LIMIT) {
                                                atomicExch(error_flag, 2);
                                                gave_up = true;
                                            } else if ((spins & 255u) == 0 && *reinterpret_cast<volatile int *>(error_flag) != 0) {
                                                gave_up = true;
                                            }
                                        }
                                        part = __uint_as_float(static_cast<uint32_t>(got));
                                    }
                                    total += part;
                                }
                            }
                            // linear + residual_add (add_bf16.comp.template:17-24): bf16(bf16(product) + residual), in place
                            a.buffers.hidden[static_cast<size_t>(epilogue_m) * shape.hidden + column] =
                                static_cast<uint16_t>(f32_to_bf16_bits(round_bf16(total) + bf16_bits_to_f32(round == 0 ? done.payload[0] : (round == 1 ? done.payload[1] : (round == 2 ? done.payload[2] : done.payload[3])))));
                        }
                    }
                }
            }
            if constexpr (EXCHANGE) {
                if (phase == 1 || phase == 3) tag += 1u;
            }
            stamp(layer, 4 * phase + 2);
            if (layer + 1 < a.layer_count || phase < 3) meet();
            stamp(layer, 4 * phase + 3);

            if (phase == 0) {
                // ---- attention: (kv head, split, stream x lane group) items, one team of four warps each, spread
                // over the SMs first; the teams' shared arrays reuse the fragment area (nothing is staged right now)
                const int streams = lanes / a.lanes_per_stream;
                const int group_slots = streams * ((a.lanes_per_stream + QL - 1) / QL);
                const int total = shape.kv_heads * a.max_splits * group_slots;
                const int team = warp >> 2;
                unsigned long long *item_stamps = (a.buffers.timing != nullptr && blockIdx.x == 0 && threadIdx.x == 0) ? a.buffers.timing + layer * 32 : nullptr;
                for (int item = blockIdx.x + gridDim.x * team; item < total; item += gridDim.x * 4)
                    attention_team_item<HD, GROUP, QL>(*attention_cache, spec->kv, item, smem_raw, item_stamps);
                consumer_sync();
                stamp(layer, 17);
                {
                    // merge the heads whose last split was completed here: one (lane, q head) row per warp and round
                    int requests = attention_cache->merge_count;
                    if (requests > ATTENTION_MERGE_LIST) requests = ATTENTION_MERGE_LIST;
                    if (requests > 0) {
                        __threadfence();
                        const int groups_per_stream = (a.lanes_per_stream + QL - 1) / QL;
                        for (int index = warp; index < requests * QL * GROUP; index += CONSUMER_WARPS) {
                            const int request = attention_cache->merge_list[index / (QL * GROUP)], row = index % (QL * GROUP);
                            const int kv_head = request / group_slots, group_slot = request % group_slots;
                            const int group_index = group_slot % groups_per_stream;
                            const int query_lane = (group_slot / groups_per_stream) * a.lanes_per_stream + group_index * QL + row / GROUP;
                            if (query_lane < lanes && group_index * QL + row / GROUP < a.lanes_per_stream && attention_cache->slot[query_lane] >= 0)
                                attention_merge_row<HD>(attention_cache->job, attention_own_splits(attention_cache->job, kv.capacity, attention_cache->tick[query_lane]),
                                                        query_lane, kv_head * GROUP + row % GROUP);
                        }
                    }
                }
                if (a.max_splits > MERGE_BLOCK) {
                    // ---- groups of more than MERGE_BLOCK splits: every warp of the grid merges ranges of MERGE_BLOCK
                    // splits into one partial each, then one warp per row merges the row's range partials.  The two
                    // barriers in between are not counted for the producer of slices (it waits for the one below).
                    const int ranges = attention_ranges(a.max_splits), rows = lanes * shape.q_heads;
                    grid_barrier(counter, target, error_flag, barrier_spin_limit);
                    for (int task = blockIdx.x + gridDim.x * warp; task < rows * ranges; task += gridDim.x * CONSUMER_WARPS) {
                        const int row = task / ranges, range = task % ranges, query_lane = row / shape.q_heads;
                        if (attention_cache->slot[query_lane] < 0) continue;
                        const int splits = attention_group_splits(attention_cache->job, attention_cache->tick, kv.capacity, query_lane, QL);
                        if (splits > MERGE_BLOCK && range * MERGE_BLOCK < splits)
                            attention_merge_range<HD>(attention_cache->job, splits, query_lane, row % shape.q_heads, range);
                    }
                    grid_barrier(counter, target, error_flag, barrier_spin_limit);
                    for (int row = blockIdx.x + gridDim.x * warp; row < rows; row += gridDim.x * CONSUMER_WARPS) {
                        const int query_lane = row / shape.q_heads;
                        if (attention_cache->slot[query_lane] < 0) continue;
                        const int splits = attention_group_splits(attention_cache->job, attention_cache->tick, kv.capacity, query_lane, QL);
                        if (splits > MERGE_BLOCK) attention_merge_ranges<HD>(attention_cache->job, splits, query_lane, row % shape.q_heads);
                    }
                }
                meet();
                if (threadIdx.x == 0) attention_cache->merge_count = 0;  // read again after the next layer's q/k/v barrier at the earliest
                stamp(layer, 18);
            }
        }
    }

    if (a.buffers.timing != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        a.buffers.timing[30] = now;
    }
    // The last CTA to leave rearms the barrier words for the next launch (every CTA has passed its last barrier
    // before it counts itself out).
    if (threadIdx.x == 0) {
        const unsigned int gone = atomicAdd(counter + 1, 1u);
        if (gone == gridDim.x - 1) {
            counter[0] = 0u;
            counter[1] = 0u;
            if constexpr (EXCHANGE) a.tp->counter[a.tp->rank][STACK_TP_WORD_CONSUMED] = tag;  // the next launch counts on from here
            __threadfence();
        }
    }
}

struct StackPlanSmem {
    size_t scratch, total;
    int stages, stage_bytes, steps_per_stage, slice_slots, slice_bytes;
};

template <int HD>
bool plan_smem_for(const StackShape &shape, int lanes, int grid, StackPlanSmem *plan) {
    const int staged = lanes < 8 ? lanes : 8;
    const int q_width = shape.q_heads * shape.head_width;
    const MatrixSchedule o = stack_schedule(shape.hidden >> 4, q_width >> 7, 1, grid);
    const MatrixSchedule down = stack_schedule(shape.hidden >> 4, shape.ffn >> 7, 1, grid);
    const int slice_groups = o.width > down.width ? o.width : down.width;
    // two steps per stage: fewer hand-overs, two blocks per warp and wait, and the gate/up step in pairs - for every
    // lane count alike, so that the order of a lane's additions does not depend on how many lanes share its launch
    const int steps_per_stage = 2;
    const size_t slice = static_cast<size_t>(steps_per_stage) * slice_groups * staged * 256;
    size_t scratch = static_cast<size_t>(staged) * shape.hidden * 2;  // fragments of a normalised row set
    const size_t teams = 4 * attention_team_bytes<HD>();
    if (teams > scratch) scratch = teams;
    if (2 * slice > scratch) scratch = 2 * slice;
    // the up rows' partial sums of the gate/up pairs sit behind the normalised rows (one copy at least)
    const size_t pairs = static_cast<size_t>(staged) * shape.hidden * 2 + CONSUMER_WARPS * 128 * sizeof(float);
    if (pairs > scratch) scratch = pairs;
    scratch = (scratch + 127) & ~static_cast<size_t>(127);
    int slice_slots = static_cast<int>(scratch / slice);
    if (slice_slots > MAX_STAGES) slice_slots = MAX_STAGES;
    const size_t fixed = scratch + 2 * CONSUMER_WARPS * 128 * sizeof(float) + 4 * CONSUMER_WARPS * sizeof(float) + 8 * (HD / 2) * sizeof(uint32_t) +
                         sizeof(AttentionCache) + 4 * sizeof(PhaseInfo) + 4 * MAX_STAGES * sizeof(uint64_t) + 4 * sizeof(uint32_t) + 128;
    const size_t stage = (static_cast<size_t>(steps_per_stage) * STAGE_WEIGHT_BYTES + 127) & ~static_cast<size_t>(127);
    const size_t limit = 227 * 1024;
    if (fixed + 2 * stage > limit) return false;
    int stages = static_cast<int>((limit - fixed) / stage);
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    plan->scratch = scratch;
    plan->stages = stages;
    plan->stage_bytes = static_cast<int>(stage);
    plan->steps_per_stage = steps_per_stage;
    plan->slice_slots = slice_slots;
    plan->slice_bytes = static_cast<int>(slice);
    plan->total = fixed + static_cast<size_t>(stages) * stage;
    return true;
}

bool plan_smem(const StackShape &shape, int lanes, int grid, StackPlanSmem *plan) {
    const int group = shape.kv_heads > 0 ? shape.q_heads / shape.kv_heads : 0;
    if (shape.head_width == 128 && (group == 4 || group == 8)) return plan_smem_for<128>(shape, lanes, grid, plan);
    if (shape.head_width == 64 && group == 4) return plan_smem_for<64>(shape, lanes, grid, plan);
    if (shape.head_width == 32 && group == 2) return plan_smem_for<32>(shape, lanes, grid, plan);
    return false;
}

template <int HD, int GROUP, bool EXCHANGE>
cudaError_t launch_instance_of(const StackArgs &args, size_t smem, int grid, cudaStream_t stream) {
    // the attribute is per device and per kernel instance: set it on every launch (a cheap host-side call)
    cudaError_t status = cudaFuncSetAttribute(decode_stack_kernel<HD, GROUP, EXCHANGE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (status != cudaSuccess) return status;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(grid);
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
cudaError_t launch_instance(const StackArgs &args, size_t smem, int grid, cudaStream_t stream) {
    return args.tp_size > 1 ? launch_instance_of<HD, GROUP, true>(args, smem, grid, stream) : launch_instance_of<HD, GROUP, false>(args, smem, grid, stream);
}

}  // namespace

size_t int4_cta_stream_bytes(int rows, int k, bool pair, int grid) {
    return stack_stream_bytes(stack_schedule(rows / 16, k / 128, pair ? 2 : 1, grid));
}

cudaError_t launch_int4_cta_streams(const RelayoutSegment *segments, int count, bool pair, int k, int grid, uint8_t *out, cudaStream_t stream) {
    if (count < 1 || count > 3 || (pair && count != 2) || k % 128 != 0 || grid < 1) return cudaErrorInvalidValue;
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
    args.schedule = stack_schedule(tiles, k / 128, pair ? 2 : 1, grid);
    const int passes = ((tiles + grid - 1) / grid + args.schedule.slots - 1) / args.schedule.slots;
    if (tiles == 0) return cudaSuccess;
    int4_cta_stream_kernel<<<dim3(passes * args.schedule.steps, grid), 256, 0, stream>>>(args, out);
    return cudaGetLastError();
}

bool decode_stack_supported(const StackShape &shape, int lanes, size_t *smem_bytes) {
    if (lanes < 1 || lanes > 8 || shape.grid < 1) return false;
    if (shape.hidden > 2 * 8 * CONSUMER_THREADS || shape.hidden % 128 != 0 || shape.ffn % 128 != 0 || (shape.q_heads * shape.head_width) % 128 != 0) return false;
    if (((shape.q_heads + 2 * shape.kv_heads) * shape.head_width) % 16 != 0) return false;
    StackPlanSmem plan;
    if (!plan_smem(shape, lanes, shape.grid, &plan)) return false;
    if (smem_bytes) *smem_bytes = plan.total;
    return true;
}

cudaError_t launch_decode_stack(const StackLayer *layers_device, int layer_count, const StackShape &shape,
                                const StackBuffers &buffers, const LaneTable &lanes_meta, int lanes, int lanes_per_stream,
                                int split_tokens, int max_splits, cudaStream_t stream, const StackTp *tp_device, int tp_size) {
    StackPlanSmem plan;
    if (lanes < 1 || lanes > 8 || !plan_smem(shape, lanes, shape.grid, &plan) || lanes_per_stream <= 0 || lanes % lanes_per_stream != 0 ||
        layer_count < 1 || split_tokens != 64 || max_splits > MERGE_BLOCK * MERGE_BLOCK)
        return cudaErrorInvalidValue;
    StackArgs args;
    args.layers = layers_device;
    args.layer_count = layer_count;
    args.shape = shape;
    args.buffers = buffers;
    args.lanes_meta = lanes_meta;
    args.lanes = lanes;
    args.lanes_per_stream = lanes_per_stream;
    args.max_splits = max_splits;
    if (tp_size < 1 || tp_size > STACK_TP_MAX_RANKS || (tp_size > 1 && tp_device == nullptr)) return cudaErrorInvalidValue;
    args.tp = tp_size > 1 ? tp_device : nullptr;
    args.tp_size = tp_size;
    args.stages = plan.stages;
    args.stage_bytes = plan.stage_bytes;
    args.steps_per_stage = plan.steps_per_stage;
    args.slice_slots = plan.slice_slots;
    args.slice_bytes = plan.slice_bytes;
    args.scratch_bytes = static_cast<uint32_t>(plan.scratch);
    args.prefetch_stages = 0;  // stages beyond the ring the producer would ask L2 for: measured, no gain
    args.debug_flags = 0;      // probe switches of the kernel (1: no hand-over checks, 4: weight stream off after the ring has filled)
    const int group = shape.q_heads / shape.kv_heads;
    if (shape.head_width == 128 && group == 4) return launch_instance<128, 4>(args, plan.total, shape.grid, stream);
    if (shape.head_width == 128 && group == 8) return launch_instance<128, 8>(args, plan.total, shape.grid, stream);
    if (shape.head_width == 64 && group == 4) return launch_instance<64, 4>(args, plan.total, shape.grid, stream);
    return launch_instance<32, 2>(args, plan.total, shape.grid, stream);
}

}  // namespace nerve

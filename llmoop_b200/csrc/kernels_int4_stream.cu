// INT4 g128 weight-streaming linear, bulk-copy pipelined (the production path for K % 1024 == 0).
//
// Why a second kernel: a warp that loads its weights with ordinary loads can keep only what its registers hold
// in flight, and a CTA that lives for one 16-row tile spends most of its life ramping up and draining.  Here
//   * CTAs are persistent (two per SM) and walk a static list of 16-row tiles;
//   * one producer warp streams the packed weights into a ring of shared-memory stages with
//     cp.async.bulk (1 KB of each weight row per 2048-column chunk - DRAM is read in page-sized contiguous
//     runs, which matters: 512-byte pieces of a row fetched microseconds apart measured ~40 % slower),
//     completion on an mbarrier, so up to STAGES x 16 KB per CTA are in flight regardless of what the consumers
//     are doing, and the stream continues across tile boundaries while the previous tile is reduced and stored;
//   * sixteen consumer warps each own one 128-column group of every chunk: they copy their 64 B x 16 rows from
//     the stage to registers, release the stage, dequantise (one lop3 per nibble pair, exact) and issue mma.sync
//     m16n8k16 bf16 -> f32 against the activation fragment, then apply the group scale to the f32 partial;
//   * weights never depend on the kernel's predecessor, so the producer starts before griddepcontrol.wait.
// Stage rows are padded by 64 B: the 16-byte reads of a quarter-warp (2 rows x 4 column pieces) then fall into
// eight distinct bank groups.
//
// Every wait on an mbarrier is bounded; on expiry the CTA raises *error_flag, stops consuming and the producer
// waits (bounded) for its outstanding copies before the CTA exits.
#include "common.cuh"
#include "kernels.cuh"

namespace nerve {

namespace {

constexpr int CONSUMER_WARPS = 16;  // warp w owns 128-column group w of every 2048-column chunk
constexpr int STREAM_THREADS = (CONSUMER_WARPS + 1) * 32;
constexpr int TILE_ROWS = 16;                      // one m16 MMA tile of weight rows
constexpr int CHUNK_COLUMNS = 2048;                // 16 groups of 128
constexpr int CHUNK_ROW_BYTES = CHUNK_COLUMNS / 2;  // 1024 contiguous bytes per row and chunk
constexpr int STAGE_ROW_STRIDE = CHUNK_ROW_BYTES + 64;
constexpr int STAGE_SCALE_OFFSET = TILE_ROWS * STAGE_ROW_STRIDE;          // group scales of the chunk: [16 rows][16 groups] bf16
constexpr int STAGE_SCALE_ROW_BYTES = (CHUNK_COLUMNS / 128) * 2;           // 32
constexpr int STAGE_BYTES = STAGE_SCALE_OFFSET + TILE_ROWS * STAGE_SCALE_ROW_BYTES;  // 17920
constexpr int STAGES = 4;
constexpr uint32_t SPIN_LIMIT = 1u << 16;  // x up to ~20 us per try: about a second

struct StreamBranch {
    const uint32_t *qweight;
    const uint16_t *scales;
    uint16_t *y;
    int n;
    int first_tile;
};

struct StreamLaunch {
    StreamBranch branch[3];
    int branches;
    int total_tiles;
    const uint16_t *x;
    const uint16_t *residual;
    int lanes;
    int k;
    int epilogue;
    int *error_flag;
};

__device__ __forceinline__ uint32_t smem_u32(const void *pointer) { return static_cast<uint32_t>(__cvta_generic_to_shared(pointer)); }

__device__ __forceinline__ void mbarrier_init(uint64_t *barrier, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(barrier)), "r"(count));
}
__device__ __forceinline__ void mbarrier_expect_tx(uint64_t *barrier, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(barrier)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbarrier_arrive(uint64_t *barrier) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(barrier)) : "memory");
}
__device__ __forceinline__ bool mbarrier_try_wait(uint64_t *barrier, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(smem_u32(barrier)), "r"(parity), "r"(20000u)  // the thread may be suspended up to ~20 us per try
        : "memory");
    return done != 0;
}
// Bounded wait: false when the limit ran out.
__device__ __forceinline__ bool mbarrier_wait(uint64_t *barrier, uint32_t parity, uint32_t limit) {
    for (uint32_t spin = 0; spin < limit; spin++)
        if (mbarrier_try_wait(barrier, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_copy_g2s(void *destination, const void *source, uint32_t bytes, uint64_t *barrier) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(destination)),
                 "l"(source), "r"(bytes), "r"(smem_u32(barrier))
                 : "memory");
}
__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_WARPS * 32) : "memory"); }

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Two nibbles (bits s..s+3 and s+16..s+19) -> bf16x2 (128+q, 128+q'), exact, one lop3.  The weight is q-8, so
// every product carries an extra 136*x; it is removed by one more MMA per k-step whose A operand is the
// constant -136 (the correction is the same for all 32 rows of the tile, so it is computed once per item and
// added to both row tiles).  This trades 64 sub.bf16x2 per item for 8 MMAs + 8 adds: the kernel is limited by
// instruction issue, not by the tensor pipe.
__device__ __forceinline__ uint32_t dequant2(uint32_t word, int shift) {
    uint32_t biased;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(biased) : "r"(word >> shift), "n"(0x000F000F), "n"(0x43004300));
    return biased;
}
constexpr uint32_t MINUS_136_BF16X2 = 0xC308C308u;

struct TileRef {
    int branch;    // branch the tile's rows belong to (SILU_PAIR: 0 = gate; the up rows are branch 1, same rows)
    int row_base;  // first weight row of the tile inside its branch
};

template <bool SILU_PAIR>
__device__ __forceinline__ TileRef locate_tile(const StreamLaunch &p, int tile) {
    TileRef ref;
    if (SILU_PAIR) {
        ref.branch = 0;
        ref.row_base = tile * TILE_ROWS;
        return ref;
    }
    int b = 0;
    if (p.branches > 1 && tile >= p.branch[1].first_tile) b = 1;
    if (p.branches > 2 && tile >= p.branch[2].first_tile) b = 2;
    ref.branch = b;
    ref.row_base = (tile - p.branch[b].first_tile) * TILE_ROWS;
    return ref;
}

__device__ __forceinline__ int clamp_row(const StreamBranch &branch, int row) { return row < branch.n ? row : branch.n - 1; }

}  // namespace

// SILU_PAIR: every tile is streamed twice over - the 16 gate rows, then the same 16 rows of the up matrix -
// and the epilogue of the second pass combines them: bf16(silu_bf16(bf16 gate) * bf16 up).
template <bool SILU_PAIR>
__global__ void __launch_bounds__(STREAM_THREADS, 2)
linear_int4_stream_kernel(const StreamLaunch p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t *stage_base = smem;                                                // STAGES x STAGE_BYTES
    float *reduce = reinterpret_cast<float *>(smem + STAGES * STAGE_BYTES);    // 2 x [16 groups][16 rows][8 lanes]
    uint64_t *full = reinterpret_cast<uint64_t *>(reduce + 2 * CONSUMER_WARPS * TILE_ROWS * 8);
    uint64_t *empty = full + STAGES;
    int *failed = reinterpret_cast<int *>(empty + STAGES);
    constexpr int PASSES = SILU_PAIR ? 2 : 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k = p.k;
    const int chunks = k / CHUNK_COLUMNS;
    const int row_bytes = k >> 1;
    const int groups = k >> 7;
    const int m0 = blockIdx.y * 8;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbarrier_init(&full[s], 1);
            mbarrier_init(&empty[s], CONSUMER_WARPS);
        }
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == CONSUMER_WARPS) {
        // ------------------------------------------------------------------ producer warp
        // lane l copies half a row piece: row l/2 of the tile, bytes (l&1)*512 .. +512 of the 1 KB chunk piece
        int item = 0;
        for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x) {
            const TileRef ref = locate_tile<SILU_PAIR>(p, tile);
            for (int pass = 0; pass < PASSES; pass++) {
                const StreamBranch &source = p.branch[SILU_PAIR ? pass : ref.branch];
                const int row = clamp_row(source, ref.row_base + (lane >> 1));  // clamped rows are computed and dropped
                const uint8_t *row_pointer =
                    reinterpret_cast<const uint8_t *>(source.qweight) + static_cast<size_t>(row) * row_bytes + (lane & 1) * (CHUNK_ROW_BYTES / 2);
                const uint16_t *scale_pointer = source.scales + static_cast<size_t>(clamp_row(source, ref.row_base + (lane & 15))) * groups;
                for (int chunk = 0; chunk < chunks; chunk++, item++) {
                    const int slot = item % STAGES;
                    const uint32_t phase = (item / STAGES) & 1;
                    bool ok = true;
                    if (lane == 0) {
                        ok = mbarrier_wait(&empty[slot], phase ^ 1u, *failed ? 16u : SPIN_LIMIT);
                        if (ok) mbarrier_expect_tx(&full[slot], TILE_ROWS * (CHUNK_ROW_BYTES + STAGE_SCALE_ROW_BYTES));
                    }
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) {
                        if (lane == 0) {
                            *failed = 1;
                            if (p.error_flag) atomicExch(p.error_flag, 1);
                        }
                        goto producer_drain;
                    }
                    bulk_copy_g2s(stage_base + slot * STAGE_BYTES + (lane >> 1) * STAGE_ROW_STRIDE + (lane & 1) * (CHUNK_ROW_BYTES / 2),
                                  row_pointer + chunk * CHUNK_ROW_BYTES, CHUNK_ROW_BYTES / 2, &full[slot]);
                    // the chunk's group scales ride in the same stage: a scale fetched by the consumers with an
                    // ordinary load would put a full DRAM latency on the critical path of every item
                    if (lane < TILE_ROWS)
                        bulk_copy_g2s(stage_base + slot * STAGE_BYTES + STAGE_SCALE_OFFSET + lane * STAGE_SCALE_ROW_BYTES,
                                      scale_pointer + chunk * (CHUNK_COLUMNS / 128), STAGE_SCALE_ROW_BYTES, &full[slot]);
                }
            }
        }
    producer_drain:
        // After a failure, copies already issued must land before the CTA's shared memory is released.
        if (lane == 0 && *failed) {
            for (int s = 0; s < STAGES; s++) (void)mbarrier_wait(&full[s], 0, 64u), (void)mbarrier_wait(&full[s], 1, 64u);
        }
        return;
    }

    // ---------------------------------------------------------------------- consumer warps
    const int g = lane >> 2, j = lane & 3;
    const bool lane_active = m0 + g < p.lanes;
    const uint16_t *xrow = p.x + static_cast<size_t>(lane_active ? m0 + g : 0) * k + warp * 128 + j * 32;
    grid_dependency_wait();  // activations (and the residual) come from the previous kernel

    int item = 0;
    int buffer = 0;
    for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x) {
        const TileRef ref = locate_tile<SILU_PAIR>(p, tile);
        float gate_value = 0.0f;  // SILU_PAIR: epilogue threads carry the gate sum from pass 0 to pass 1
        for (int pass = 0; pass < PASSES; pass++, buffer ^= 1) {
            const StreamBranch &source = p.branch[SILU_PAIR ? pass : ref.branch];
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};

            for (int chunk = 0; chunk < chunks; chunk++, item++) {
                const int slot = item % STAGES;
                const uint32_t phase = (item / STAGES) & 1;
                // activation fragment and scales first: they do not depend on the stage
                uint32_t bfrag[8][2];
                if (lane_active) {
#pragma unroll
                    for (int word = 0; word < 4; word++) {
                        const uint4 xv = __ldg(reinterpret_cast<const uint4 *>(xrow + chunk * CHUNK_COLUMNS) + word);
                        bfrag[2 * word][0] = __byte_perm(xv.x, xv.z, 0x5410);      // (v0, v4)
                        bfrag[2 * word][1] = __byte_perm(xv.x, xv.z, 0x7632);      // (v1, v5)
                        bfrag[2 * word + 1][0] = __byte_perm(xv.y, xv.w, 0x5410);  // (v2, v6)
                        bfrag[2 * word + 1][1] = __byte_perm(xv.y, xv.w, 0x7632);  // (v3, v7)
                    }
                } else {
#pragma unroll
                    for (int step = 0; step < 8; step++) bfrag[step][0] = bfrag[step][1] = 0u;
                }

                // offset correction -136 * sum_k x[m][k] over this group seeds the accumulator
                float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int step = 0; step < 8; step++)
                    mma_16816(c, MINUS_136_BF16X2, MINUS_136_BF16X2, MINUS_136_BF16X2, MINUS_136_BF16X2, bfrag[step][0], bfrag[step][1]);

                bool ok = true;
                if (lane == 0) ok = mbarrier_wait(&full[slot], phase, *failed ? 16u : SPIN_LIMIT);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) {
                    if (lane == 0) {
                        *failed = 1;
                        if (p.error_flag) atomicExch(p.error_flag, 1);
                    }
                    continue;  // keep the barrier protocol moving; results of this launch are invalid
                }
                const uint8_t *stage = stage_base + slot * STAGE_BYTES + warp * 64 + j * 16;
                const uint4 wqa = *reinterpret_cast<const uint4 *>(stage + g * STAGE_ROW_STRIDE);
                const uint4 wqb = *reinterpret_cast<const uint4 *>(stage + (g + 8) * STAGE_ROW_STRIDE);
                const uint16_t *stage_scales = reinterpret_cast<const uint16_t *>(stage_base + slot * STAGE_BYTES + STAGE_SCALE_OFFSET) + warp;
                const float scale_a = bf16_bits_to_f32(stage_scales[g * (CHUNK_COLUMNS / 128)]);
                const float scale_b = bf16_bits_to_f32(stage_scales[(g + 8) * (CHUNK_COLUMNS / 128)]);
                __syncwarp();
                if (lane == 0) mbarrier_arrive(&empty[slot]);

                const uint32_t wa[4] = {wqa.x, wqa.y, wqa.z, wqa.w};
                const uint32_t wb[4] = {wqb.x, wqb.y, wqb.z, wqb.w};
#pragma unroll
                for (int word = 0; word < 4; word++) {
                    mma_16816(c, dequant2(wa[word], 0), dequant2(wb[word], 0), dequant2(wa[word], 4), dequant2(wb[word], 4),
                              bfrag[2 * word][0], bfrag[2 * word][1]);
                    mma_16816(c, dequant2(wa[word], 8), dequant2(wb[word], 8), dequant2(wa[word], 12), dequant2(wb[word], 12),
                              bfrag[2 * word + 1][0], bfrag[2 * word + 1][1]);
                }
                acc[0] = fmaf(c[0], scale_a, acc[0]);
                acc[1] = fmaf(c[1], scale_a, acc[1]);
                acc[2] = fmaf(c[2], scale_b, acc[2]);
                acc[3] = fmaf(c[3], scale_b, acc[3]);
            }

            // ---- cross-warp reduction of the pass (double-buffered so that one barrier per pass suffices)
            float *partial = reduce + buffer * (CONSUMER_WARPS * TILE_ROWS * 8);
            {
                float *rows = partial + warp * TILE_ROWS * 8;
                rows[g * 8 + 2 * j] = acc[0];
                rows[g * 8 + 2 * j + 1] = acc[1];
                rows[(g + 8) * 8 + 2 * j] = acc[2];
                rows[(g + 8) * 8 + 2 * j + 1] = acc[3];
            }
            consumer_barrier();
            if (threadIdx.x < TILE_ROWS * 8) {
                const int local_row = threadIdx.x >> 3, m = threadIdx.x & 7;
                const int row = ref.row_base + local_row;
                if (m0 + m < p.lanes && row < source.n) {
                    float sum = 0.0f;
#pragma unroll
                    for (int w = 0; w < CONSUMER_WARPS; w++) sum += partial[(w * TILE_ROWS + local_row) * 8 + m];
                    const size_t out = static_cast<size_t>(m0 + m) * source.n + row;
                    if (SILU_PAIR) {
                        if (pass == 0) {
                            gate_value = sum;
                        } else {
                            float value = rounded_silu(round_bf16(gate_value)) * round_bf16(sum);
                            p.branch[2].y[out] = static_cast<uint16_t>(f32_to_bf16_bits(value));
                        }
                    } else {
                        if (p.epilogue == EPILOGUE_RESIDUAL_ROUNDED) sum = round_bf16(sum) + bf16_bits_to_f32(p.residual[out]);
                        else if (p.epilogue == EPILOGUE_RESIDUAL_F32) sum = sum + bf16_bits_to_f32(p.residual[out]);
                        source.y[out] = static_cast<uint16_t>(f32_to_bf16_bits(sum));
                    }
                }
            }
        }
    }
    grid_launch_dependents();
}

namespace {

size_t stream_smem_bytes() { return static_cast<size_t>(STAGES) * STAGE_BYTES + 2 * CONSUMER_WARPS * TILE_ROWS * 8 * sizeof(float) + 2 * STAGES * 8 + 16; }

template <bool SILU_PAIR>
cudaError_t launch_stream(const StreamLaunch &params, int lane_tiles, cudaStream_t stream) {
    static bool configured = false;
    static int sm_count = 0;
    const size_t smem = stream_smem_bytes();
    if (!configured) {
        cudaError_t status = cudaFuncSetAttribute(linear_int4_stream_kernel<SILU_PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                  static_cast<int>(smem));
        if (status != cudaSuccess) return status;
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
        configured = true;
    }
    // persistent grid: two CTAs per SM (shared memory allows two), never more CTAs than tiles
    int ctas = sm_count * 2;
    if (ctas > params.total_tiles) ctas = params.total_tiles;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(ctas, lane_tiles);
    config.blockDim = dim3(STREAM_THREADS);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, linear_int4_stream_kernel<SILU_PAIR>, params);
}

}  // namespace

bool linear_int4_stream_supported(int k) { return k > 0 && k % CHUNK_COLUMNS == 0; }

cudaError_t launch_linear_int4_stream(const uint16_t *x, int branches, const uint32_t *const *qweights, const uint16_t *const *scales,
                                      uint16_t *const *ys, const int *ns, const uint16_t *residual, int lanes, int k, int epilogue,
                                      int *error_flag, cudaStream_t stream) {
    StreamLaunch params = {};
    params.branches = branches;
    params.x = x;
    params.residual = residual;
    params.lanes = lanes;
    params.k = k;
    params.epilogue = epilogue;
    params.error_flag = error_flag;
    int tiles = 0;
    for (int b = 0; b < branches; b++) {
        params.branch[b] = StreamBranch{qweights[b], scales[b], ys[b], ns[b], tiles};
        tiles += (ns[b] + TILE_ROWS - 1) / TILE_ROWS;
    }
    params.total_tiles = tiles;
    return launch_stream<false>(params, (lanes + 7) / 8, stream);
}

cudaError_t launch_linear_int4_stream_silu_pair(const uint16_t *x, const uint32_t *gate_q, const uint16_t *gate_s, const uint32_t *up_q,
                                                const uint16_t *up_s, uint16_t *y, int lanes, int n, int k, int *error_flag,
                                                cudaStream_t stream) {
    StreamLaunch params = {};
    params.branches = 2;
    params.x = x;
    params.lanes = lanes;
    params.k = k;
    params.error_flag = error_flag;
    params.branch[0] = StreamBranch{gate_q, gate_s, nullptr, n, 0};
    params.branch[1] = StreamBranch{up_q, up_s, nullptr, n, 0};
    params.branch[2] = StreamBranch{nullptr, nullptr, y, n, 0};
    params.total_tiles = (n + TILE_ROWS - 1) / TILE_ROWS;
    return launch_stream<true>(params, (lanes + 7) / 8, stream);
}

}  // namespace nerve

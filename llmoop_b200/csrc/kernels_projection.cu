// Output projection (logits = scale * normalised hidden . table^T, f32: tied_output_projection_batch_bf16.comp.template:52-142)
// for a handful of lanes over a vocabulary-sized bf16 table - 1 GB for the 8B configuration, read four times per
// speculative cycle - as a persistent streaming kernel: one CTA per SM, a producer thread that keeps a ring of bulk
// asynchronous copies of the table in flight, eight consumer warps on the tensor cores.
//
// The table is read from a copy made at mount in the order the consumers use it: for every tile of 16 rows and every
// chunk of 32 columns, 1 KB holding, for each thread (g, j) of a warp, the 16 bytes of row g and of row g + 8 at
// columns 8 j .. 8 j + 7 of the chunk.  A tile is therefore contiguous (K / 32 KB) and a ring stage is one bulk copy.
// The eight values a thread holds feed two mma.sync.m16n8k16 as they come (the k slots of an MMA may be permuted at
// will as long as A and B agree), against the same 16 bytes of the lane's activation row.  Warp w of a CTA takes the
// chunks w, w + 8, ... of a tile; the eight partial sums meet in shared memory once per tile.
#include "common.cuh"
#include "kernels.cuh"

namespace nerve {

namespace {

constexpr int PROJECTION_WARPS = 8;
constexpr int PROJECTION_THREADS = PROJECTION_WARPS * 32 + 32;  // + the producer warp
constexpr int PROJECTION_STAGE_CHUNKS = 32;                    // chunks of 32 columns per ring stage: 32 KB
constexpr int PROJECTION_STAGE_BYTES = PROJECTION_STAGE_CHUNKS * 1024;
constexpr int PROJECTION_STAGES = 6;
constexpr unsigned int PROJECTION_SPIN_LIMIT = 1u << 18;  // attempts of about 20 us each

__global__ void projection_table_kernel(const uint16_t *__restrict__ table, uint4 *__restrict__ out, int rows, int k) {
    const int chunks = k / 32;
    const size_t total = static_cast<size_t>((rows + 15) / 16) * chunks * 64;
    for (size_t index = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; index < total; index += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int lane = static_cast<int>(index & 31), half = static_cast<int>((index >> 5) & 1);
        const size_t rest = index >> 6;
        const int chunk = static_cast<int>(rest % chunks);
        const int tile = static_cast<int>(rest / chunks);
        const int row = tile * 16 + (lane >> 2) + 8 * half;
        uint4 value = make_uint4(0, 0, 0, 0);
        if (row < rows) value = *reinterpret_cast<const uint4 *>(table + static_cast<size_t>(row) * k + chunk * 32 + (lane & 3) * 8);
        out[index] = value;
    }
}

__device__ __forceinline__ void projection_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ bool projection_wait(uint32_t barrier, uint32_t parity, int *error_flag) {
    unsigned int spins = 0;
    while (true) {
        uint32_t done;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(done)
            : "r"(barrier), "r"(parity), "r"(20000u)
            : "memory");
        if (done) return true;
        if (++spins > PROJECTION_SPIN_LIMIT) {
            if (error_flag != nullptr) atomicExch(error_flag, 3);
            return false;
        }
        if (error_flag != nullptr && (spins & 255u) == 0 && *reinterpret_cast<volatile int *>(error_flag) != 0) return false;
    }
}

struct ProjectionArgs {
    const uint16_t *x;      // [lanes][k] normalised rows
    const uint4 *table;     // the mount-time copy, first tile of the slice to project
    float *logits;          // [lanes][rows] f32 * scale, or ...
    uint16_t *rounded;      // ... [lanes][rows] bf16(sum) when this is set (a plain bf16 linear)
    int lanes, rows, k;     // rows of the slice (output row stride)
    float scale;
    int *error_flag;
};

__global__ void __launch_bounds__(PROJECTION_THREADS, 1) output_projection_kernel(const ProjectionArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *barriers = reinterpret_cast<uint64_t *>(smem);                        // full[STAGES], empty[STAGES]
    float *reduce = reinterpret_cast<float *>(smem + 128);                          // [2][8 warps][16 rows][8 lanes]
    uint8_t *ring = smem + 128 + 2 * PROJECTION_WARPS * 128 * sizeof(float);
    const uint32_t full = static_cast<uint32_t>(__cvta_generic_to_shared(barriers)), empty = full + PROJECTION_STAGES * 8;
    const uint32_t ring_address = static_cast<uint32_t>(__cvta_generic_to_shared(ring));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, j = lane & 3;
    const int chunks = a.k / 32, tiles = (a.rows + 15) / 16;
    const int stages_per_tile = (chunks + PROJECTION_STAGE_CHUNKS - 1) / PROJECTION_STAGE_CHUNKS;
    const int my_tiles = tiles > static_cast<int>(blockIdx.x) ? (tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x) : 0;
    if (threadIdx.x == 0) {
        for (int s = 0; s < PROJECTION_STAGES; s++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(full + s * 8) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(empty + s * 8), "r"(PROJECTION_WARPS) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async;" ::: "memory");
    }
    __syncthreads();

    if (warp == PROJECTION_WARPS) {
        if (lane != 0) return;
        uint32_t slot = 0, parity = 1;
        for (int t = 0; t < my_tiles; t++) {
            const uint8_t *source = reinterpret_cast<const uint8_t *>(a.table) + (static_cast<size_t>(blockIdx.x) + static_cast<size_t>(t) * gridDim.x) * chunks * 1024;
            for (int s = 0; s < stages_per_tile; s++) {
                const int first = s * PROJECTION_STAGE_CHUNKS;
                const uint32_t bytes = static_cast<uint32_t>((chunks - first < PROJECTION_STAGE_CHUNKS ? chunks - first : PROJECTION_STAGE_CHUNKS) * 1024);
                if (!projection_wait(empty + slot * 8, parity, a.error_flag)) {
                    for (int i = 0; i < 64; i++) __nanosleep(1000);  // let the copies in flight land before the shared memory goes away
                    return;
                }
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full + slot * 8), "r"(bytes) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(ring_address + slot * PROJECTION_STAGE_BYTES),
                             "l"(__cvta_generic_to_global(source + static_cast<size_t>(first) * 1024)), "r"(bytes), "r"(full + slot * 8)
                             : "memory");
                if (++slot == PROJECTION_STAGES) {
                    slot = 0;
                    parity ^= 1u;
                }
            }
        }
        return;
    }

    // ---- consumers
    const int lane_row = g < a.lanes ? g : a.lanes - 1;  // lanes beyond the batch repeat the last one; their columns are dropped
    const uint4 *x_row = reinterpret_cast<const uint4 *>(a.x + static_cast<size_t>(lane_row) * a.k) + j;
    uint32_t slot = 0, parity = 0;
    int buffer = 0;
    bool alive = true;  // once a wait has expired the rest runs without waiting (garbage, reported through the error word)
    for (int t = 0; t < my_tiles; t++) {
        float acc[2][4] = {};
        for (int s = 0; s < stages_per_tile; s++) {
            const int first = s * PROJECTION_STAGE_CHUNKS;
            const int count = chunks - first < PROJECTION_STAGE_CHUNKS ? chunks - first : PROJECTION_STAGE_CHUNKS;
            if (alive && !projection_wait(full + slot * 8, parity, a.error_flag)) alive = false;
            const uint4 *stage = reinterpret_cast<const uint4 *>(ring + static_cast<size_t>(slot) * PROJECTION_STAGE_BYTES);
#pragma unroll 4
            for (int c = warp; c < count; c += PROJECTION_WARPS) {
                const uint4 low = stage[c * 64 + lane], high = stage[c * 64 + 32 + lane];
                const uint4 xv = __ldg(x_row + (first + c) * 4);
                projection_mma(acc[0], low.x, high.x, low.y, high.y, xv.x, xv.y);
                projection_mma(acc[1], low.z, high.z, low.w, high.w, xv.z, xv.w);
            }
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty + slot * 8) : "memory");
            if (++slot == PROJECTION_STAGES) {
                slot = 0;
                parity ^= 1u;
            }
        }
        // the warps' partial sums meet: (row g | g + 8, lanes 2j, 2j + 1) per thread
        float *mine = reduce + static_cast<size_t>(buffer * PROJECTION_WARPS + warp) * 128;
        *reinterpret_cast<float2 *>(mine + g * 8 + 2 * j) = make_float2(acc[0][0] + acc[1][0], acc[0][1] + acc[1][1]);
        *reinterpret_cast<float2 *>(mine + (g + 8) * 8 + 2 * j) = make_float2(acc[0][2] + acc[1][2], acc[0][3] + acc[1][3]);
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (threadIdx.x < 128) {
            const int row = threadIdx.x >> 3, m = threadIdx.x & 7;
            const float *source = reduce + static_cast<size_t>(buffer * PROJECTION_WARPS) * 128 + row * 8 + m;
            float sum = 0.0f;
#pragma unroll
            for (int w = 0; w < PROJECTION_WARPS; w++) sum += source[w * 128];
            const int out_row = (static_cast<int>(blockIdx.x) + t * static_cast<int>(gridDim.x)) * 16 + row;
            if (m < a.lanes && out_row < a.rows) {
                if (a.rounded != nullptr) a.rounded[static_cast<size_t>(m) * a.rows + out_row] = static_cast<uint16_t>(f32_to_bf16_bits(sum));
                else a.logits[static_cast<size_t>(m) * a.rows + out_row] = sum * a.scale;
            }
        }
        buffer ^= 1;  // the next tile's partial sums go to the other half; this one is read until the next barrier at the latest
    }
}

}  // namespace

size_t projection_table_bytes(int rows, int k) { return static_cast<size_t>((rows + 15) / 16) * (k / 32) * 1024; }

cudaError_t launch_projection_table(const uint16_t *table, void *out, int rows, int k, cudaStream_t stream) {
    if (k % 32 != 0 || rows < 1) return cudaErrorInvalidValue;
    projection_table_kernel<<<1024, 256, 0, stream>>>(table, static_cast<uint4 *>(out), rows, k);
    return cudaGetLastError();
}

bool output_projection_supported(int lanes, int k) { return lanes >= 1 && lanes <= 8 && k % 32 == 0; }

cudaError_t launch_output_projection(const uint16_t *x, const void *streamed_table, int first_row, float *logits, int lanes, int rows, int k, float scale,
                                     int grid, int *error_flag, cudaStream_t stream, uint16_t *rounded) {
    if (lanes <= 0 || rows <= 0) return cudaSuccess;
    if (!output_projection_supported(lanes, k) || first_row % 16 != 0 || grid < 1) return cudaErrorInvalidValue;
    const size_t smem = 128 + 2 * PROJECTION_WARPS * 128 * sizeof(float) + static_cast<size_t>(PROJECTION_STAGES) * PROJECTION_STAGE_BYTES;
    cudaError_t status = cudaFuncSetAttribute(output_projection_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (status != cudaSuccess) return status;
    ProjectionArgs args;
    args.x = x;
    args.table = reinterpret_cast<const uint4 *>(static_cast<const uint8_t *>(streamed_table) + static_cast<size_t>(first_row / 16) * (k / 32) * 1024);
    args.logits = logits;
    args.rounded = rounded;
    args.lanes = lanes;
    args.rows = rows;
    args.k = k;
    args.scale = scale;
    args.error_flag = error_flag;
    output_projection_kernel<<<grid, PROJECTION_THREADS, smem, stream>>>(args);
    return cudaGetLastError();
}

}  // namespace nerve

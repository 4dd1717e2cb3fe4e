// bf16 linear for batches of 16 lanes and more (the draft adapter's linear over a prefill chunk, the output
// projection of a many-stream verify batch) on the fifth-generation tensor cores: y[m][n] = sum_k x[m][k] * w[n][k],
// the arithmetic of linear_bf16.comp.template / tied_output_projection_batch_bf16.comp.template:52-142 (bf16
// operands, f32 accumulation, one rounding or the logit scale at the end).
//
// One CTA computes a 128 (weight rows) x 64 (lanes) tile.  Weight rows are the M side of tcgen05.mma, lanes its N
// side; both operands sit in shared memory in the K-major core-matrix layout (8 rows x 16 bytes per core matrix, no
// swizzle) and the f32 accumulator stays in tensor memory over the whole of K - unlike the INT4 kernel there is no
// per-group scale to apply, so nothing is read back until the end.  Four stages of (128 x 128 weights, 64 x 128
// activations) are filled with 16-byte asynchronous copies by all threads, three K blocks ahead; one thread issues
// the eight MMAs of a block (K = 16 each) and commits them to the stage's mbarrier, which is what allows the stage
// to be filled again.  Waits are bounded; a wait that expires sets the error word, and the CTA still frees its
// tensor memory before it leaves.
#include "common.cuh"
#include "kernels.cuh"

namespace nerve {

namespace {

constexpr int BGEMM_ROWS = 128;   // weight rows per CTA (MMA M)
constexpr int BGEMM_LANES = 64;   // lanes per CTA (MMA N)
constexpr int BGEMM_THREADS = 256;
constexpr int BGEMM_STAGES = 4;
constexpr int BGEMM_A_BYTES = BGEMM_ROWS * 128 * 2;   // one K block of 128 of a row block
constexpr int BGEMM_B_BYTES = BGEMM_LANES * 128 * 2;
constexpr int BGEMM_STAGE_BYTES = BGEMM_A_BYTES + BGEMM_B_BYTES;
constexpr int BGEMM_BLOCK_STRIDE = 16 * 128;          // bytes between 8-row blocks: 16 core matrices of a block's K
constexpr unsigned int BGEMM_SPIN_LIMIT = 1u << 22;
constexpr size_t BGEMM_SMEM = static_cast<size_t>(BGEMM_STAGES) * BGEMM_STAGE_BYTES + 128;

// tcgen05.mma kind::f16 instruction descriptor: f32 accumulator, A and B bf16, both K-major, N / 8 in bits 17-22,
// M / 16 in bits 24-28.
constexpr uint32_t BGEMM_INSTRUCTION = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BGEMM_LANES / 8) << 17) |
                                       (static_cast<uint32_t>(BGEMM_ROWS / 16) << 24);

// Shared-memory matrix descriptor, K-major without swizzle (start address / 16, the distance between the two core
// matrices of a K = 16 step, the distance between 8-row blocks, descriptor version 1).
__device__ __forceinline__ uint64_t bgemm_descriptor(uint32_t shared_address) {
    return static_cast<uint64_t>((shared_address & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(128 >> 4) << 16) |
           (static_cast<uint64_t>(BGEMM_BLOCK_STRIDE >> 4) << 32) | (1ull << 46);
}

__device__ __forceinline__ bool bgemm_wait(uint32_t barrier, uint32_t parity, int *error_flag) {
    unsigned int spins = 0;
    while (true) {
        uint32_t done;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(done)
            : "r"(barrier), "r"(parity)
            : "memory");
        if (done) return true;
        if (++spins > BGEMM_SPIN_LIMIT) {
            if (error_flag != nullptr) atomicExch(error_flag, 3);
            return false;
        }
    }
}

struct BgemmArgs {
    const uint16_t *x, *w;
    void *y;
    const uint16_t *residual;
    int lanes, n, k, epilogue;
    float scale;
    int *error_flag;
};

__global__ void __launch_bounds__(BGEMM_THREADS) linear_bf16_gemm_kernel(const BgemmArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *barriers = reinterpret_cast<uint64_t *>(smem + static_cast<size_t>(BGEMM_STAGES) * BGEMM_STAGE_BYTES);  // one per stage, then the last one
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(barriers + BGEMM_STAGES + 1);
    const uint32_t barrier_address = static_cast<uint32_t>(__cvta_generic_to_shared(barriers));
    const uint32_t tiles = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * BGEMM_LANES, row0 = blockIdx.y * BGEMM_ROWS;
    const int blocks = a.k >> 7;

    if (threadIdx.x == 0) {
        for (int s = 0; s <= BGEMM_STAGES; s++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(barrier_address + s * 8) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {  // 64 columns of tensor memory: one accumulator
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(tmem_slot))), "r"(64u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(tmem_slot);

    // copy roles: thread t moves the eight 16-byte pieces of half `t & 1` of weight row `t >> 1` and four 16-byte
    // pieces of the activations; rows and lanes beyond the matrix repeat the last one (their results are not stored)
    const int fetch_row = threadIdx.x >> 1, fetch_half = threadIdx.x & 1;
    const int weight_row = row0 + fetch_row < a.n ? row0 + fetch_row : a.n - 1;
    const uint16_t *weight_source = a.w + static_cast<size_t>(weight_row) * a.k + fetch_half * 64;
    const uint32_t weight_offset = static_cast<uint32_t>((fetch_row >> 3) * BGEMM_BLOCK_STRIDE + fetch_half * 8 * 128 + (fetch_row & 7) * 16);
    auto fill = [&](int block) {
        const uint32_t stage = tiles + static_cast<uint32_t>(block % BGEMM_STAGES) * BGEMM_STAGE_BYTES;
        const uint16_t *source = weight_source + static_cast<size_t>(block) * 128;
#pragma unroll
        for (int piece = 0; piece < 8; piece++)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(stage + weight_offset + piece * 128), "l"(source + piece * 8) : "memory");
#pragma unroll
        for (int i = 0; i < BGEMM_LANES * 16 / BGEMM_THREADS; i++) {
            const int piece = threadIdx.x + i * BGEMM_THREADS, n = piece >> 4, part = piece & 15;
            const int m = m0 + n < a.lanes ? m0 + n : a.lanes - 1;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(stage + BGEMM_A_BYTES + (n >> 3) * BGEMM_BLOCK_STRIDE + part * 128 + (n & 7) * 16),
                         "l"(a.x + static_cast<size_t>(m) * a.k + block * 128 + part * 8)
                         : "memory");
        }
    };

    bool alive = true;
    for (int block = 0; block < BGEMM_STAGES - 1; block++) {
        if (block < blocks) fill(block);
        asm volatile("cp.async.commit_group;" ::: "memory");  // one group per K block, also when it is empty
    }
    for (int block = 0; block < blocks && alive; block++) {
        // the stage of block + STAGES - 1 is the one block - 1 was multiplied from: filled again once those MMAs are done
        if (block >= 1 && block + BGEMM_STAGES - 1 < blocks) {
            const int previous = block - 1;
            if (!bgemm_wait(barrier_address + (previous % BGEMM_STAGES) * 8, static_cast<uint32_t>((previous / BGEMM_STAGES) & 1), a.error_flag)) alive = false;
        }
        if (block + BGEMM_STAGES - 1 < blocks) fill(block + BGEMM_STAGES - 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group %0;" ::"n"(BGEMM_STAGES - 1) : "memory");  // this block's copies have landed
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");                 // ... and the tensor core may read them
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (threadIdx.x == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_address = tiles + static_cast<uint32_t>(block % BGEMM_STAGES) * BGEMM_STAGE_BYTES, b_address = a_address + BGEMM_A_BYTES;
#pragma unroll
            for (int step = 0; step < 8; step++) {  // K = 16 per instruction: two core matrices = 256 bytes further per step
                const uint64_t a_descriptor = bgemm_descriptor(a_address + step * 256), b_descriptor = bgemm_descriptor(b_address + step * 256);
                const uint32_t accumulate = (block > 0 || step > 0) ? 1u : 0u;
                asm volatile(
                    "{\n"
                    ".reg .pred p;\n"
                    "setp.ne.b32 p, %4, 0;\n"
                    "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n"
                    "}\n" ::"r"(tmem_base),
                    "l"(a_descriptor), "l"(b_descriptor), "r"(BGEMM_INSTRUCTION), "r"(accumulate), "r"(0u)
                    : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(barrier_address + (block % BGEMM_STAGES) * 8) : "memory");
            if (block == blocks - 1)
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(barrier_address + BGEMM_STAGES * 8) : "memory");
        }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    // ---- epilogue: thread = row 32 * (warp & 3) + lane of the tile, columns 32 * (warp >> 2) .. + 31
    if (alive && blocks > 0 && !bgemm_wait(barrier_address + BGEMM_STAGES * 8, 0u, a.error_flag)) alive = false;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int out_row = 32 * (warp & 3) + lane, column0 = 32 * (warp >> 2);
    if (alive && blocks > 0) {
        const uint32_t address = tmem_base + (static_cast<uint32_t>(32 * (warp & 3)) << 16) + static_cast<uint32_t>(column0);
#pragma unroll
        for (int half = 0; half < 2; half++) {
            uint32_t d[16];
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                         : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7]), "=r"(d[8]), "=r"(d[9]),
                           "=r"(d[10]), "=r"(d[11]), "=r"(d[12]), "=r"(d[13]), "=r"(d[14]), "=r"(d[15])
                         : "r"(address + half * 16)
                         : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (row0 + out_row < a.n) {
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const int m = m0 + column0 + half * 16 + i;
                    if (m >= a.lanes) break;
                    const size_t index = static_cast<size_t>(m) * a.n + row0 + out_row;
                    float sum = __uint_as_float(d[i]);
                    if (a.epilogue == EPILOGUE_F32_SCALED) {
                        reinterpret_cast<float *>(a.y)[index] = sum * a.scale;
                    } else {
                        if (a.epilogue == EPILOGUE_RESIDUAL_ROUNDED) sum = round_bf16(sum) + bf16_bits_to_f32(a.residual[index]);
                        else if (a.epilogue == EPILOGUE_RESIDUAL_F32) sum = sum + bf16_bits_to_f32(a.residual[index]);
                        reinterpret_cast<uint16_t *>(a.y)[index] = static_cast<uint16_t>(f32_to_bf16_bits(sum));
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(64u) : "memory");
}

}  // namespace

// From 16 lanes on (a quarter of the tile's lane side) the table is better read once than once per eight lanes.
bool linear_bf16_gemm_supported(int lanes, int n, int k) { return lanes >= BGEMM_LANES / 4 && k % 128 == 0 && k >= 128 && n >= 1; }

cudaError_t launch_linear_bf16_gemm(const uint16_t *x, const uint16_t *w, void *y, const uint16_t *residual, int lanes, int n, int k, int epilogue,
                                    float scale, int *error_flag, cudaStream_t stream) {
    if (lanes <= 0) return cudaSuccess;
    if (!linear_bf16_gemm_supported(lanes, n, k)) return cudaErrorInvalidValue;
    cudaError_t status = cudaFuncSetAttribute(linear_bf16_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(BGEMM_SMEM));
    if (status != cudaSuccess) return status;
    BgemmArgs args{x, w, y, residual, lanes, n, k, epilogue, scale, error_flag};
    dim3 grid((lanes + BGEMM_LANES - 1) / BGEMM_LANES, (n + BGEMM_ROWS - 1) / BGEMM_ROWS);
    linear_bf16_gemm_kernel<<<grid, BGEMM_THREADS, BGEMM_SMEM, stream>>>(args);
    return cudaGetLastError();
}

}  // namespace nerve

// INT4 g128 weight-only linear for batches of 64 lanes and more (prefill chunks, wide verify batches) on the
// fifth-generation tensor cores: y[m][n] = sum_k x[m][k] * (q[n][k] - 8) * scale[n][k / 128], the arithmetic of
// linear_int4_ct.comp.template:80-150 with the tile-level structure of the reference's prefill kernel
// (linear_batch_cooperative_int4.comp.template:78-212).
//
// One CTA computes a 128 (weight rows) x 64 (lanes) tile.  The weight rows are the M side of tcgen05.mma, the lanes
// its N side; both operands are bf16 in shared memory in the K-major core-matrix layout (8 rows x 16 bytes per core
// matrix, no swizzle), the f32 accumulator lives in tensor memory.  Per quantisation group of 128 columns:
//   1. all 256 threads fetch the group's packed nibbles (64 bytes per row) and the lanes' activations, turn the
//      nibbles into exact bf16 (q - 8) - lop3 into the mantissa of 128.0, subtract 136 - and store both tiles; the
//      eight values of a 16-byte piece sit in the order (0,4,1,5,2,6,3,7) on both sides, which the contraction
//      does not see;
//   2. one thread issues eight tcgen05.mma (K = 16 each) into one of two accumulator buffers, starting it from zero,
//      and commits them to an mbarrier;
//   3. while the tensor core works on this group, the threads read the previous group's accumulator back
//      (tcgen05.ld, one row per thread), multiply it by the row's group scale and add it to f32 registers - the
//      reference's order: f32 sum inside a group, one multiplication by the scale, f32 sum over the groups.
// Shared-memory tiles and accumulators are double-buffered, so fetching, the MMAs and the scaling of three
// consecutive groups overlap.  Waits are bounded; a wait that expires sets the error word, and the CTA still frees
// its tensor memory before it leaves.
#include "common.cuh"
#include "kernels.cuh"

namespace nerve {

namespace {

constexpr int GEMM_ROWS = 128;     // weight rows per CTA (MMA M)
constexpr int GEMM_MIN_LANES = 64; // lanes per CTA (MMA N): 64, or 128 for batches of 128 lanes and more - the weights
                                   // are then dequantised once per 128 lanes
constexpr int GEMM_THREADS = 256;
constexpr int GEMM_A_BYTES = GEMM_ROWS * 128 * 2;    // one group of a row block, bf16
constexpr int GEMM_BLOCK_STRIDE = 16 * 128;          // bytes between 8-row blocks: 16 core matrices of a group's K
constexpr unsigned int GEMM_SPIN_LIMIT = 1u << 22;
template <int LANES>
constexpr size_t gemm_smem() { return 2 * (GEMM_A_BYTES + LANES * 128 * 2) + 64; }

// 32-bit instruction descriptor of tcgen05.mma kind::f16: f32 accumulator (bits 4-5 = 1), A and B bf16 (bits 7-9 and
// 10-12 = 1), both K-major (bits 15, 16 = 0), N / 8 in bits 17-22, M / 16 in bits 24-28.
template <int LANES>
constexpr uint32_t gemm_instruction() {
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(LANES / 8) << 17) | (static_cast<uint32_t>(GEMM_ROWS / 16) << 24);
}

// Shared-memory matrix descriptor, K-major without swizzle: start address / 16 in bits 0-13, the byte distance
// between the two core matrices of a K = 16 step (128) / 16 in bits 16-29, the distance between 8-row blocks / 16 in
// bits 32-45, descriptor version 1 in bits 46-47.
__device__ __forceinline__ uint64_t matrix_descriptor(uint32_t shared_address) {
    return static_cast<uint64_t>((shared_address & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(128 >> 4) << 16) |
           (static_cast<uint64_t>(GEMM_BLOCK_STRIDE >> 4) << 32) | (1ull << 46);
}

// Two nibbles (bits s..s+3 and s+16..s+19 of `word`) -> bf16x2 (q - 8, q' - 8), exact.
__device__ __forceinline__ uint32_t nibble_pair_bf16(uint32_t word, int shift) {
    uint32_t biased, out;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(biased) : "r"(word >> shift), "n"(0x000F000F), "n"(0x43004300));
    asm("sub.bf16x2 %0, %1, %2;" : "=r"(out) : "r"(biased), "r"(0x43084308u));
    return out;
}

__device__ __forceinline__ bool wait_barrier(uint32_t barrier, uint32_t parity, int *error_flag) {
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
        if (++spins > GEMM_SPIN_LIMIT) {
            if (error_flag != nullptr) atomicExch(error_flag, 3);
            return false;
        }
    }
}

struct GemmArgs {
    const uint16_t *x;
    const uint32_t *qweights[3];  // up to three matrices that share the activations (q, k, v) in one launch:
    const uint16_t *scale_rows[3];
    void *ys[3];
    int ns[3];
    int first_tile[4];            // ... matrix b owns the row tiles first_tile[b] .. first_tile[b + 1] - 1 of the grid
    const uint16_t *residual;
    int lanes, k, epilogue;
    float scale;
    int *error_flag;
};
struct GemmMatrix {  // the matrix a CTA works on
    const uint32_t *qweight;
    const uint16_t *scales;
    void *y;
    int n;
};

template <int GEMM_LANES>
__global__ void __launch_bounds__(GEMM_THREADS) linear_int4_gemm_kernel(const GemmArgs a) {
    constexpr int GEMM_B_BYTES = GEMM_LANES * 128 * 2;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t *tile_a[2] = {smem, smem + GEMM_A_BYTES + GEMM_B_BYTES};
    uint8_t *tile_b[2] = {smem + GEMM_A_BYTES, smem + 2 * GEMM_A_BYTES + GEMM_B_BYTES};
    uint64_t *barriers = reinterpret_cast<uint64_t *>(smem + 2 * (GEMM_A_BYTES + GEMM_B_BYTES));
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(barriers + 2);
    const uint32_t barrier_address = static_cast<uint32_t>(__cvta_generic_to_shared(barriers));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int branch = 0;
    while (branch < 2 && static_cast<int>(blockIdx.y) >= a.first_tile[branch + 1]) branch++;
    GemmMatrix matrix;  // the same fields under the names the single-matrix kernel used: a.qweight, a.scales, a.y, a.n
    matrix.qweight = a.qweights[branch];
    matrix.scales = a.scale_rows[branch];
    matrix.y = a.ys[branch];
    matrix.n = a.ns[branch];
    const int m0 = blockIdx.x * GEMM_LANES, row0 = (static_cast<int>(blockIdx.y) - a.first_tile[branch]) * GEMM_ROWS;
    const int groups = a.k >> 7, words_per_row = a.k >> 3;

    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(barrier_address) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(barrier_address + 8) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {  // two accumulators of LANES columns of tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(tmem_slot))), "r"(static_cast<uint32_t>(2 * GEMM_LANES))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(tmem_slot);

    // fetch roles: thread t turns the 64 nibbles of half `t & 1` of row `t >> 1` into eight 16-byte pieces, and
    // moves four 16-byte pieces of the activations
    const int fetch_row = threadIdx.x >> 1, fetch_half = threadIdx.x & 1;
    const int weight_row = row0 + fetch_row < matrix.n ? row0 + fetch_row : matrix.n - 1;
    const uint4 *weight_source = reinterpret_cast<const uint4 *>(matrix.qweight + static_cast<size_t>(weight_row) * words_per_row) + fetch_half * 2;
    const uint32_t weight_offset = static_cast<uint32_t>((fetch_row >> 3) * GEMM_BLOCK_STRIDE + fetch_half * 8 * 128 + (fetch_row & 7) * 16);
    // accumulator roles: thread = row 32 * (warp & 3) + lane of the tile, one half of the tile's columns
    constexpr int COLUMNS = GEMM_LANES / 2;
    const int out_row = 32 * (warp & 3) + lane, column0 = COLUMNS * (warp >> 2);
    const uint16_t *scale_row = matrix.scales + static_cast<size_t>(row0 + out_row < matrix.n ? row0 + out_row : matrix.n - 1) * groups;
    float acc[COLUMNS];
#pragma unroll
    for (int i = 0; i < COLUMNS; i++) acc[i] = 0.0f;
    bool alive = true;

    // The packed nibbles and the activations of a group are requested one group ahead (into registers) and turned
    // into the shared-memory tiles when their turn comes, so the memory latency of group g + 1 hides behind the
    // MMAs of group g and the scaling of group g - 1.
    uint4 raw_weights[2], raw_x[GEMM_LANES * 16 / GEMM_THREADS];
    auto request = [&](int group) {
        raw_weights[0] = __ldg(weight_source + group * 4);
        raw_weights[1] = __ldg(weight_source + group * 4 + 1);
#pragma unroll
        for (int i = 0; i < GEMM_LANES * 16 / GEMM_THREADS; i++) {
            const int piece = threadIdx.x + i * GEMM_THREADS, n = piece >> 4, block = piece & 15;
            raw_x[i] = make_uint4(0, 0, 0, 0);
            if (m0 + n < a.lanes) raw_x[i] = __ldg(reinterpret_cast<const uint4 *>(a.x + static_cast<size_t>(m0 + n) * a.k + group * 128) + block);
        }
    };
    auto store_tiles = [&](int buffer) {
        const uint32_t words[8] = {raw_weights[0].x, raw_weights[0].y, raw_weights[0].z, raw_weights[0].w,
                                   raw_weights[1].x, raw_weights[1].y, raw_weights[1].z, raw_weights[1].w};
        uint8_t *destination = tile_a[buffer] + weight_offset;
#pragma unroll
        for (int w = 0; w < 8; w++)
            *reinterpret_cast<uint4 *>(destination + w * 128) = make_uint4(nibble_pair_bf16(words[w], 0), nibble_pair_bf16(words[w], 4),
                                                                           nibble_pair_bf16(words[w], 8), nibble_pair_bf16(words[w], 12));
#pragma unroll
        for (int i = 0; i < GEMM_LANES * 16 / GEMM_THREADS; i++) {
            const int piece = threadIdx.x + i * GEMM_THREADS, n = piece >> 4, block = piece & 15;
            const uint4 raw = raw_x[i];
            // (x0,x1)(x2,x3)(x4,x5)(x6,x7) -> (x0,x4)(x1,x5)(x2,x6)(x3,x7): the order the nibble pairs come out in
            const uint4 ordered = make_uint4(__byte_perm(raw.x, raw.z, 0x5410), __byte_perm(raw.x, raw.z, 0x7632), __byte_perm(raw.y, raw.w, 0x5410),
                                             __byte_perm(raw.y, raw.w, 0x7632));
            *reinterpret_cast<uint4 *>(tile_b[buffer] + (n >> 3) * GEMM_BLOCK_STRIDE + block * 128 + (n & 7) * 16) = ordered;
        }
    };
    // adds scale(group) x the accumulator of `buffer` to the registers
    auto drain = [&](int group, int buffer) {
        if (!wait_barrier(barrier_address + buffer * 8, static_cast<uint32_t>((group >> 1) & 1), a.error_flag)) alive = false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const float scale = bf16_bits_to_f32(scale_row[group]);
        const uint32_t address = tmem_base + (static_cast<uint32_t>(32 * (warp & 3)) << 16) + static_cast<uint32_t>(buffer * GEMM_LANES + column0);
#pragma unroll
        for (int half = 0; half < COLUMNS / 16; half++) {
            uint32_t d[16];
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                         : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7]), "=r"(d[8]), "=r"(d[9]),
                           "=r"(d[10]), "=r"(d[11]), "=r"(d[12]), "=r"(d[13]), "=r"(d[14]), "=r"(d[15])
                         : "r"(address + half * 16)
                         : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int i = 0; i < 16; i++) acc[half * 16 + i] = fmaf(scale, __uint_as_float(d[i]), acc[half * 16 + i]);
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    };

    if (groups > 0) request(0);
    for (int group = 0; group < groups && alive; group++) {
        const int buffer = group & 1;
        store_tiles(buffer);  // the MMAs that read this buffer two groups ago were waited for in the last drain
        if (group + 1 < groups) request(group + 1);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the tiles were written with ordinary stores; the tensor core reads them
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (threadIdx.x == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_address = static_cast<uint32_t>(__cvta_generic_to_shared(tile_a[buffer]));
            const uint32_t b_address = static_cast<uint32_t>(__cvta_generic_to_shared(tile_b[buffer]));
            const uint32_t d_address = tmem_base + static_cast<uint32_t>(buffer * GEMM_LANES);
#pragma unroll
            for (int step = 0; step < 8; step++) {  // K = 16 per instruction: two core matrices = 256 bytes further per step
                const uint64_t a_descriptor = matrix_descriptor(a_address + step * 256), b_descriptor = matrix_descriptor(b_address + step * 256);
                const uint32_t accumulate = step > 0 ? 1u : 0u;
                asm volatile(
                    "{\n"
                    ".reg .pred p;\n"
                    "setp.ne.b32 p, %4, 0;\n"
                    "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n"
                    "}\n" ::"r"(d_address),
                    "l"(a_descriptor), "l"(b_descriptor), "r"(gemm_instruction<GEMM_LANES>()), "r"(accumulate), "r"(0u)
                    : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(barrier_address + buffer * 8) : "memory");
        }
        if (group > 0) drain(group - 1, buffer ^ 1);
    }
    if (alive && groups > 0) drain(groups - 1, (groups - 1) & 1);

    // ---- epilogue: this thread's row, 32 lanes
    if (alive && row0 + out_row < matrix.n) {
#pragma unroll
        for (int i = 0; i < COLUMNS; i++) {
            const int m = m0 + column0 + i;
            if (m >= a.lanes) break;
            const size_t index = static_cast<size_t>(m) * matrix.n + row0 + out_row;
            float sum = acc[i];
            if (a.epilogue == EPILOGUE_F32_SCALED) {
                reinterpret_cast<float *>(matrix.y)[index] = sum * a.scale;
            } else {
                if (a.epilogue == EPILOGUE_RESIDUAL_ROUNDED) sum = round_bf16(sum) + bf16_bits_to_f32(a.residual[index]);
                else if (a.epilogue == EPILOGUE_RESIDUAL_F32) sum = sum + bf16_bits_to_f32(a.residual[index]);
                reinterpret_cast<uint16_t *>(matrix.y)[index] = static_cast<uint16_t>(f32_to_bf16_bits(sum));
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(static_cast<uint32_t>(2 * GEMM_LANES)) : "memory");
}

}  // namespace

bool linear_int4_gemm_supported(int lanes, int n, int k) { return lanes >= GEMM_MIN_LANES && k % 128 == 0 && k >= 128 && n >= 1; }

cudaError_t launch_linear_int4_gemm_multi(const uint16_t *x, int branches, const uint32_t *const *qweights, const uint16_t *const *scales, void *const *ys,
                                          const int *ns, const uint16_t *residual, int lanes, int k, int epilogue, float scale, int *error_flag,
                                          cudaStream_t stream) {
    if (lanes <= 0) return cudaSuccess;
    if (branches < 1 || branches > 3 || (residual != nullptr && branches != 1)) return cudaErrorInvalidValue;
    GemmArgs args = {};
    args.x = x;
    int tiles = 0;
    for (int b = 0; b < 3; b++) {
        const int source = b < branches ? b : branches - 1;
        if (b < branches && !linear_int4_gemm_supported(lanes, ns[b], k)) return cudaErrorInvalidValue;
        args.qweights[b] = qweights[source];
        args.scale_rows[b] = scales[source];
        args.ys[b] = ys[source];
        args.ns[b] = ns[source];
        args.first_tile[b] = tiles;
        if (b < branches) tiles += (ns[b] + GEMM_ROWS - 1) / GEMM_ROWS;
    }
    args.first_tile[3] = tiles;
    for (int b = branches; b < 3; b++) args.first_tile[b] = tiles;  // no tile belongs to an absent matrix
    args.residual = residual;
    args.lanes = lanes;
    args.k = k;
    args.epilogue = epilogue;
    args.scale = scale;
    args.error_flag = error_flag;
    if (lanes >= 128) {
        cudaError_t status = cudaFuncSetAttribute(linear_int4_gemm_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(gemm_smem<128>()));
        if (status != cudaSuccess) return status;
        linear_int4_gemm_kernel<128><<<dim3((lanes + 127) / 128, tiles), GEMM_THREADS, gemm_smem<128>(), stream>>>(args);
    } else {
        cudaError_t status = cudaFuncSetAttribute(linear_int4_gemm_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(gemm_smem<64>()));
        if (status != cudaSuccess) return status;
        linear_int4_gemm_kernel<64><<<dim3((lanes + 63) / 64, tiles), GEMM_THREADS, gemm_smem<64>(), stream>>>(args);
    }
    return cudaGetLastError();
}

cudaError_t launch_linear_int4_gemm(const uint16_t *x, const uint32_t *qweight, const uint16_t *scales, void *y, const uint16_t *residual, int lanes,
                                    int n, int k, int epilogue, float scale, int *error_flag, cudaStream_t stream) {
    return launch_linear_int4_gemm_multi(x, 1, &qweight, &scales, &y, &n, residual, lanes, k, epilogue, scale, error_flag, stream);
}

}  // namespace nerve

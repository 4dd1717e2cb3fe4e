// Weight-streaming linears for small lane counts (verify M = k+1, draft M = 1,
// multi-stream batches): y[m][n] = sum_k x[m][k] * W[n][k].
//
// All of these are HBM-bound: every weight byte is read once per launch, the
// activations (KBs) stay in L1/L2.  Algorithmic bytes per output row:
//   INT4 g128: k/2 packed + 2*k/128 scale bytes;  BF16: 2*k;  FP8: k + block scales.
//
// INT4 path (linear_int4_ct.comp.template:80-150 semantics): at 4 lanes a
// scalar-FMA kernel needs ~6 ALU ops per nibble (unpack, offset, 4 FMAs), i.e.
// ~280 thread-ops/clk/SM to keep up with HBM, above the 128/clk an SM issues,
// so the dot products run on the tensor cores even at M <= 8:
// mma.sync.m16n8k16 with A = 16 weight rows dequantised in registers to bf16
// (exact: 128+q built with one lop3, minus 136), B = up to 8 activation lanes,
// f32 accumulators; the group scale is applied to the f32 partial after every
// 128-column group, so rounding happens only once at the bf16 store.
// The K permutation inside an mma is free as long as A and B agree: thread
// (g, j) of a warp feeds logical k slots {2j,2j+1,2j+8,2j+9} from nibbles
// {0,4,1,5} / {2,6,3,7} of its own 32-bit words, which lets each thread fetch
// 32 consecutive nibbles (one 128-bit load) per row and keeps dequantisation
// at 3 ALU ops per nibble pair.
#include <mma.h>

#include <cstdlib>

#include "common.cuh"
#include "kernels.cuh"

namespace nerve {

// ----------------------------------------------------------------------------- bf16 weights

template <int MT, int ROWS>
__global__ void __launch_bounds__(256)
linear_bf16_kernel(const uint16_t *__restrict__ x, const uint16_t *__restrict__ w, void *__restrict__ y,
                   const uint16_t *__restrict__ residual, int lanes, int n, int k, int epilogue, float scale) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = (blockIdx.x * 8 + warp) * ROWS;
    const int m0 = blockIdx.y * MT;
    if (row0 >= n) return;
    float acc[ROWS][MT];
#pragma unroll
    for (int r = 0; r < ROWS; r++)
#pragma unroll
        for (int m = 0; m < MT; m++) acc[r][m] = 0.0f;

    const int chunks = k / 8;  // uint4 = 8 bf16
    // weights do not depend on the previous kernel: the first loads may be issued before the dependency wait
    grid_dependency_wait();
    for (int chunk = lane; chunk < chunks; chunk += 32) {
        uint4 wv[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; r++) {
            int row = row0 + r < n ? row0 + r : n - 1;
            wv[r] = __ldg(reinterpret_cast<const uint4 *>(w + static_cast<size_t>(row) * k) + chunk);
        }
#pragma unroll
        for (int m = 0; m < MT; m++) {
            if (m0 + m >= lanes) break;
            uint4 xv = __ldg(reinterpret_cast<const uint4 *>(x + static_cast<size_t>(m0 + m) * k) + chunk);
            const uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int r = 0; r < ROWS; r++) {
                const uint32_t ws[4] = {wv[r].x, wv[r].y, wv[r].z, wv[r].w};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    acc[r][m] = fmaf(bf16_lo(xs[i]), bf16_lo(ws[i]), acc[r][m]);
                    acc[r][m] = fmaf(bf16_hi(xs[i]), bf16_hi(ws[i]), acc[r][m]);
                }
            }
        }
    }
    // tail for k not a multiple of 8 (tiny test shapes)
    for (int col = chunks * 8 + lane; col < k; col += 32) {
#pragma unroll
        for (int r = 0; r < ROWS; r++) {
            int row = row0 + r < n ? row0 + r : n - 1;
            float wf = bf16_bits_to_f32(w[static_cast<size_t>(row) * k + col]);
#pragma unroll
            for (int m = 0; m < MT; m++)
                if (m0 + m < lanes) acc[r][m] = fmaf(bf16_bits_to_f32(x[static_cast<size_t>(m0 + m) * k + col]), wf, acc[r][m]);
        }
    }
#pragma unroll
    for (int r = 0; r < ROWS; r++)
#pragma unroll
        for (int m = 0; m < MT; m++) acc[r][m] = warp_sum(acc[r][m]);
    if (lane == 0) {
#pragma unroll
        for (int r = 0; r < ROWS; r++) {
            int row = row0 + r;
            if (row >= n) break;
#pragma unroll
            for (int m = 0; m < MT; m++) {
                if (m0 + m >= lanes) break;
                size_t index = static_cast<size_t>(m0 + m) * n + row;
                float sum = acc[r][m];
                if (epilogue == EPILOGUE_F32_SCALED) {
                    reinterpret_cast<float *>(y)[index] = sum * scale;
                } else {
                    if (epilogue == EPILOGUE_RESIDUAL_ROUNDED) sum = round_bf16(sum) + bf16_bits_to_f32(residual[index]);
                    else if (epilogue == EPILOGUE_RESIDUAL_F32) sum = sum + bf16_bits_to_f32(residual[index]);
                    reinterpret_cast<uint16_t *>(y)[index] = static_cast<uint16_t>(f32_to_bf16_bits(sum));
                }
            }
        }
    }
}

cudaError_t launch_linear_bf16(const uint16_t *x, const uint16_t *w, void *y, const uint16_t *residual, int lanes,
                               int n, int k, int epilogue, float scale, cudaStream_t stream, int *error_flag) {
    if (lanes <= 0) return cudaSuccess;
    // wide batches: the tensor-core GEMM (weights read once per 64 lanes instead of once per 8)
    if (linear_bf16_gemm_supported(lanes, n, k)) return launch_linear_bf16_gemm(x, w, y, residual, lanes, n, k, epilogue, scale, error_flag, stream);
    constexpr int ROWS = 4;
    int row_ctas = (n + 8 * ROWS - 1) / (8 * ROWS);
    if (lanes <= 4) {
        dim3 grid(row_ctas, 1);
        linear_bf16_kernel<4, ROWS><<<grid, 256, 0, stream>>>(x, w, y, residual, lanes, n, k, epilogue, scale);
    } else {
        dim3 grid(row_ctas, (lanes + 7) / 8);
        linear_bf16_kernel<8, ROWS><<<grid, 256, 0, stream>>>(x, w, y, residual, lanes, n, k, epilogue, scale);
    }
    return cudaGetLastError();
}

// parallel_linear_silu_multiply_bf16.comp.template:58-72
template <int MT>
__global__ void __launch_bounds__(256)
linear_silu_multiply_bf16_kernel(const uint16_t *__restrict__ x, const uint16_t *__restrict__ wg,
                                 const uint16_t *__restrict__ wu, uint16_t *__restrict__ y, int lanes, int n, int k) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * 8 + warp;
    const int m0 = blockIdx.y * MT;
    if (row >= n) return;
    float gate[MT], up[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) gate[m] = up[m] = 0.0f;
    grid_dependency_wait();
    for (int col = lane * 2; col < k; col += 64) {
        uint32_t g = *reinterpret_cast<const uint32_t *>(wg + static_cast<size_t>(row) * k + col);
        uint32_t u = *reinterpret_cast<const uint32_t *>(wu + static_cast<size_t>(row) * k + col);
#pragma unroll
        for (int m = 0; m < MT; m++) {
            if (m0 + m >= lanes) break;
            uint32_t xv = *reinterpret_cast<const uint32_t *>(x + static_cast<size_t>(m0 + m) * k + col);
            gate[m] = fmaf(bf16_lo(xv), bf16_lo(g), gate[m]);
            gate[m] = fmaf(bf16_hi(xv), bf16_hi(g), gate[m]);
            up[m] = fmaf(bf16_lo(xv), bf16_lo(u), up[m]);
            up[m] = fmaf(bf16_hi(xv), bf16_hi(u), up[m]);
        }
    }
#pragma unroll
    for (int m = 0; m < MT; m++) {
        gate[m] = warp_sum(gate[m]);
        up[m] = warp_sum(up[m]);
    }
    if (lane == 0)
#pragma unroll
        for (int m = 0; m < MT; m++) {
            if (m0 + m >= lanes) break;
            float value = rounded_silu(round_bf16(gate[m])) * round_bf16(up[m]);
            y[static_cast<size_t>(m0 + m) * n + row] = static_cast<uint16_t>(f32_to_bf16_bits(value));
        }
}

cudaError_t launch_linear_silu_multiply_bf16(const uint16_t *x, const uint16_t *wg, const uint16_t *wu, uint16_t *y,
                                             int lanes, int n, int k, cudaStream_t stream) {
    if (lanes <= 0) return cudaSuccess;
    dim3 grid((n + 7) / 8, (lanes + 7) / 8);
    linear_silu_multiply_bf16_kernel<8><<<grid, 256, 0, stream>>>(x, wg, wu, y, lanes, n, k);
    return cudaGetLastError();
}

// ----------------------------------------------------------------------------- INT4 g128 (tensor cores)

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Two nibbles (bits s..s+3 and s+16..s+19 of `word`) -> bf16x2 (q-8, q'-8), exact.
__device__ __forceinline__ uint32_t dequant_pair(uint32_t word, int shift) {
    uint32_t biased;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(biased) : "r"(word >> shift), "n"(0x000F000F), "n"(0x43004300));
    __nv_bfloat162 value = *reinterpret_cast<__nv_bfloat162 *>(&biased);
    const uint32_t offset_bits = 0x43084308u;  // bf16 136.0 twice
    __nv_bfloat162 offset = *reinterpret_cast<const __nv_bfloat162 *>(&offset_bits);
    value = __hsub2(value, offset);
    return *reinterpret_cast<uint32_t *>(&value);
}

struct Int4Branch {
    const uint32_t *qweight;
    const uint16_t *scales;
    uint16_t *y;
    int n;
    int first_tile;  // index of this branch's first CTA tile
};

struct Int4Launch {
    Int4Branch branch[3];
    int branches;
    const uint16_t *x;
    const uint16_t *residual;
    int lanes;
    int k;
    int epilogue;
};

constexpr int INT4_WARPS = 8;

// RT row tiles (16 rows each) per CTA; SILU_PAIR: rt 0 = gate rows, rt 1 = the same rows of the up projection,
// epilogue bf16(silu_bf16(bf16 gate) * bf16 up).  The 8 warps of a CTA split K by 128-column groups
// (warp w takes groups w, w+8, ...) and keep STAGES groups of packed weights in flight in registers: with
// ~1 us of loaded-memory latency a warp must have several KB outstanding for the SM to reach its share of HBM
// bandwidth (Little's law: ~44 KB per SM at 6.5 TB/s).
template <int RT, bool SILU_PAIR, int STAGES>
__global__ void __launch_bounds__(INT4_WARPS * 32, 2)
linear_int4_mma_kernel(const Int4Launch p) {
    __shared__ float reduce[INT4_WARPS][RT * 16][8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, j = lane & 3;
    const int m0 = blockIdx.y * 8;

    int b = 0;
    if (!SILU_PAIR) {
        if (p.branches > 1 && static_cast<int>(blockIdx.x) >= p.branch[1].first_tile) b = 1;
        if (p.branches > 2 && static_cast<int>(blockIdx.x) >= p.branch[2].first_tile) b = 2;
    }
    const Int4Branch &br = p.branch[b];
    const int tile = blockIdx.x - br.first_tile;
    const int k = p.k;
    const int words_per_row = k >> 3;
    const int groups = k >> 7;

    const uint32_t *wrow[RT][2];
    const uint16_t *srow[RT][2];
#pragma unroll
    for (int rt = 0; rt < RT; rt++) {
        const Int4Branch &source = SILU_PAIR ? p.branch[rt] : br;
        int base = SILU_PAIR ? tile * 16 : (tile * RT + rt) * 16;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            int row = base + g + 8 * h;
            if (row >= source.n) row = source.n - 1;  // clamped rows are computed and dropped
            wrow[rt][h] = source.qweight + static_cast<size_t>(row) * words_per_row + j * 4;
            srow[rt][h] = source.scales + static_cast<size_t>(row) * groups;
        }
    }
    const bool lane_active = m0 + g < p.lanes;
    const uint16_t *xrow = p.x + static_cast<size_t>(lane_active ? m0 + g : 0) * k + j * 32;

    float acc[RT][4];
#pragma unroll
    for (int rt = 0; rt < RT; rt++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[rt][i] = 0.0f;

    // Weights do not depend on the producer of x: the first STAGES groups are requested before the dependency wait.
    uint4 wq[STAGES][RT][2];
#pragma unroll
    for (int s = 0; s < STAGES; s++) {
        const int group = warp + s * INT4_WARPS;
        if (group < groups) {
#pragma unroll
            for (int rt = 0; rt < RT; rt++)
#pragma unroll
                for (int h = 0; h < 2; h++) wq[s][rt][h] = __ldg(reinterpret_cast<const uint4 *>(wrow[rt][h] + group * 16));
        }
    }
    grid_dependency_wait();

    for (int base = warp; base < groups; base += INT4_WARPS * STAGES) {
#pragma unroll
        for (int s = 0; s < STAGES; s++) {
            const int group = base + s * INT4_WARPS;
            if (group >= groups) break;
            // activations of lane g for this thread's 32 columns, permuted to match the nibble pairs
            uint32_t bfrag[8][2];
            if (lane_active) {
#pragma unroll
                for (int word = 0; word < 4; word++) {
                    uint4 xv = __ldg(reinterpret_cast<const uint4 *>(xrow + group * 128) + word);
                    bfrag[2 * word][0] = __byte_perm(xv.x, xv.z, 0x5410);      // (v0, v4)
                    bfrag[2 * word][1] = __byte_perm(xv.x, xv.z, 0x7632);      // (v1, v5)
                    bfrag[2 * word + 1][0] = __byte_perm(xv.y, xv.w, 0x5410);  // (v2, v6)
                    bfrag[2 * word + 1][1] = __byte_perm(xv.y, xv.w, 0x7632);  // (v3, v7)
                }
            } else {
#pragma unroll
                for (int step = 0; step < 8; step++) bfrag[step][0] = bfrag[step][1] = 0u;
            }
#pragma unroll
            for (int rt = 0; rt < RT; rt++) {
                float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                const uint32_t wa[4] = {wq[s][rt][0].x, wq[s][rt][0].y, wq[s][rt][0].z, wq[s][rt][0].w};
                const uint32_t wb[4] = {wq[s][rt][1].x, wq[s][rt][1].y, wq[s][rt][1].z, wq[s][rt][1].w};
#pragma unroll
                for (int word = 0; word < 4; word++) {
                    mma_bf16_16816(c, dequant_pair(wa[word], 0), dequant_pair(wb[word], 0), dequant_pair(wa[word], 4),
                                   dequant_pair(wb[word], 4), bfrag[2 * word][0], bfrag[2 * word][1]);
                    mma_bf16_16816(c, dequant_pair(wa[word], 8), dequant_pair(wb[word], 8), dequant_pair(wa[word], 12),
                                   dequant_pair(wb[word], 12), bfrag[2 * word + 1][0], bfrag[2 * word + 1][1]);
                }
                float sa = bf16_bits_to_f32(srow[rt][0][group]);
                float sb = bf16_bits_to_f32(srow[rt][1][group]);
                acc[rt][0] = fmaf(c[0], sa, acc[rt][0]);
                acc[rt][1] = fmaf(c[1], sa, acc[rt][1]);
                acc[rt][2] = fmaf(c[2], sb, acc[rt][2]);
                acc[rt][3] = fmaf(c[3], sb, acc[rt][3]);
            }
            // refill this stage's registers with the group STAGES rounds ahead
            const int next = group + INT4_WARPS * STAGES;
            if (next < groups) {
#pragma unroll
                for (int rt = 0; rt < RT; rt++)
#pragma unroll
                    for (int h = 0; h < 2; h++) wq[s][rt][h] = __ldg(reinterpret_cast<const uint4 *>(wrow[rt][h] + next * 16));
            }
        }
    }
    grid_launch_dependents();

#pragma unroll
    for (int rt = 0; rt < RT; rt++) {
        reduce[warp][rt * 16 + g][2 * j] = acc[rt][0];
        reduce[warp][rt * 16 + g][2 * j + 1] = acc[rt][1];
        reduce[warp][rt * 16 + g + 8][2 * j] = acc[rt][2];
        reduce[warp][rt * 16 + g + 8][2 * j + 1] = acc[rt][3];
    }
    __syncthreads();
    const int outputs = (SILU_PAIR ? 16 : RT * 16) * 8;
    for (int index = threadIdx.x; index < outputs; index += blockDim.x) {
        int local_row = index >> 3, m = index & 7;
        if (m0 + m >= p.lanes) continue;
        if (SILU_PAIR) {
            int row = tile * 16 + local_row;
            if (row >= br.n) continue;
            float gate = 0.0f, up = 0.0f;
#pragma unroll
            for (int w = 0; w < INT4_WARPS; w++) {
                gate += reduce[w][local_row][m];
                up += reduce[w][16 + local_row][m];
            }
            float value = rounded_silu(round_bf16(gate)) * round_bf16(up);
            p.branch[2].y[static_cast<size_t>(m0 + m) * br.n + row] = static_cast<uint16_t>(f32_to_bf16_bits(value));
        } else {
            int row = tile * RT * 16 + local_row;
            if (row >= br.n) continue;
            float sum = 0.0f;
#pragma unroll
            for (int w = 0; w < INT4_WARPS; w++) sum += reduce[w][local_row][m];
            size_t out = static_cast<size_t>(m0 + m) * br.n + row;
            if (p.epilogue == EPILOGUE_F32_SCALED) {  // f32 partial sums (tensor-parallel row split)
                reinterpret_cast<float *>(br.y)[out] = sum;
                continue;
            }
            if (p.epilogue == EPILOGUE_RESIDUAL_ROUNDED) sum = round_bf16(sum) + bf16_bits_to_f32(p.residual[out]);
            else if (p.epilogue == EPILOGUE_RESIDUAL_F32) sum = sum + bf16_bits_to_f32(p.residual[out]);
            br.y[out] = static_cast<uint16_t>(f32_to_bf16_bits(sum));
        }
    }
}

// Launch with the programmatic-dependent-launch attribute so the weight prefetch
// of this kernel overlaps the tail of the previous kernel in the stream.
template <typename Kernel>
static cudaError_t launch_pdl(Kernel kernel, dim3 grid, dim3 block, cudaStream_t stream, const Int4Launch &params) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = 0;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, kernel, params);
}

cudaError_t launch_linear_int4_multi(const uint16_t *x, int branches, const uint32_t *const *qweights,
                                     const uint16_t *const *scales, uint16_t *const *ys, const int *ns,
                                     const uint16_t *residual, int lanes, int k, int epilogue, cudaStream_t stream, int *error_flag) {
    if (lanes <= 0) return cudaSuccess;
    if (k % 128 != 0 || branches < 1 || branches > 3) return cudaErrorInvalidValue;
    if (linear_int4_gemm_supported(lanes, ns[0], k)) {
        // wide batches (prefill chunks, many-stream verify): one tcgen05 GEMM launch for all the matrices that share
        // the activations, the weights read once per 64 lanes
        for (int b = 1; b < branches; b++)
            if (!linear_int4_gemm_supported(lanes, ns[b], k)) return cudaErrorInvalidValue;
        void *outputs[3] = {ys[0], branches > 1 ? ys[1] : nullptr, branches > 2 ? ys[2] : nullptr};
        return launch_linear_int4_gemm_multi(x, branches, qweights, scales, outputs, ns, branches == 1 ? residual : nullptr, lanes, k, epilogue, 1.0f, error_flag,
                                             stream);
    }
    Int4Launch params = {};
    params.branches = branches;
    params.x = x;
    params.residual = residual;
    params.lanes = lanes;
    params.k = k;
    params.epilogue = epilogue;
    long total_rows = 0;
    for (int b = 0; b < branches; b++) total_rows += ns[b];
    const int rt = 1;
    int tiles = 0;
    for (int b = 0; b < branches; b++) {
        params.branch[b] = Int4Branch{qweights[b], scales[b], ys[b], ns[b], tiles};
        tiles += (ns[b] + 16 * rt - 1) / (16 * rt);
    }
    dim3 grid(tiles, (lanes + 7) / 8);
    return launch_pdl(linear_int4_mma_kernel<1, false, 4>, grid, dim3(INT4_WARPS * 32), stream, params);
}

cudaError_t launch_linear_int4(const uint16_t *x, const uint32_t *qweight, const uint16_t *scales, uint16_t *y,
                               const uint16_t *residual, int lanes, int n, int k, int group, int epilogue,
                               cudaStream_t stream, int *error_flag) {
    if (group != 128) return cudaErrorInvalidValue;
    return launch_linear_int4_multi(x, 1, &qweight, &scales, &y, &n, residual, lanes, k, epilogue, stream, error_flag);
}

// gate/up pair with the SiLU*up epilogue (gate -> bf16, SiLU -> bf16, up -> bf16, product -> bf16: the
// rounding chain of linear + linear + silu_multiply_bf16.comp.template:30-52).
cudaError_t launch_linear_int4_silu_pair(const uint16_t *x, const uint32_t *gate_q, const uint16_t *gate_s,
                                         const uint32_t *up_q, const uint16_t *up_s, uint16_t *y, int lanes, int n,
                                         int k, cudaStream_t stream) {
    if (lanes <= 0) return cudaSuccess;
    if (k % 128 != 0) return cudaErrorInvalidValue;
    Int4Launch params = {};
    params.branches = 2;
    params.x = x;
    params.lanes = lanes;
    params.k = k;
    params.branch[0] = Int4Branch{gate_q, gate_s, nullptr, n, 0};
    params.branch[1] = Int4Branch{up_q, up_s, nullptr, n, 0};
    params.branch[2] = Int4Branch{nullptr, nullptr, y, n, 0};
    dim3 grid((n + 15) / 16, (lanes + 7) / 8);
    return launch_pdl(linear_int4_mma_kernel<2, true, 2>, grid, dim3(INT4_WARPS * 32), stream, params);
}

// ----------------------------------------------------------------------------- FP8 W8A8 (block-scaled)

// linear_prequant_fp8_e4m3.comp.template:69-120: per 4 elements an exact f32
// dot of e4m3 values, fma'd with act_scale*weight_scale.  Here the 128-column
// block partial is accumulated first and scaled once (same value up to f32
// rounding order).  One warp per output row; lane handles 4 columns per step.
template <int MT>
__device__ __forceinline__ void fp8_row_dot(const uint8_t *__restrict__ xq, const float *__restrict__ xscale,
                                            const uint8_t *__restrict__ wrow, const uint16_t *__restrict__ wscale_row,
                                            int k, int lanes, int m0, int lane, float (&acc)[MT]) {
    const int blocks = k >> 7;
    for (int block = 0; block < blocks; block++) {
        uint32_t wpacked = __ldg(reinterpret_cast<const uint32_t *>(wrow + block * 128) + lane);
        float wf[4] = {e4m3_to_f32(wpacked & 0xff), e4m3_to_f32((wpacked >> 8) & 0xff), e4m3_to_f32((wpacked >> 16) & 0xff),
                       e4m3_to_f32(wpacked >> 24)};
        float ws = bf16_bits_to_f32(wscale_row[block]);
#pragma unroll
        for (int m = 0; m < MT; m++) {
            if (m0 + m >= lanes) break;
            uint32_t xpacked = __ldg(reinterpret_cast<const uint32_t *>(xq + static_cast<size_t>(m0 + m) * k + block * 128) + lane);
            float d = e4m3_to_f32(xpacked & 0xff) * wf[0];
            d += e4m3_to_f32((xpacked >> 8) & 0xff) * wf[1];
            d += e4m3_to_f32((xpacked >> 16) & 0xff) * wf[2];
            d += e4m3_to_f32(xpacked >> 24) * wf[3];
            acc[m] = fmaf(d, xscale[static_cast<size_t>(m0 + m) * blocks + block] * ws, acc[m]);
        }
    }
}

template <int MT>
__global__ void __launch_bounds__(256)
linear_fp8_kernel(const uint8_t *__restrict__ xq, const float *__restrict__ xscale, const uint8_t *__restrict__ w,
                  const uint16_t *__restrict__ wscale, uint16_t *__restrict__ y, const uint16_t *__restrict__ residual,
                  int lanes, int n, int k, int epilogue) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * 8 + warp;
    const int m0 = blockIdx.y * MT;
    if (row >= n) return;
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) acc[m] = 0.0f;
    grid_dependency_wait();
    fp8_row_dot<MT>(xq, xscale, w + static_cast<size_t>(row) * k, wscale + static_cast<size_t>(row >> 7) * (k >> 7), k, lanes,
                    m0, lane, acc);
#pragma unroll
    for (int m = 0; m < MT; m++) acc[m] = warp_sum(acc[m]);
    if (lane == 0)
#pragma unroll
        for (int m = 0; m < MT; m++) {
            if (m0 + m >= lanes) break;
            size_t index = static_cast<size_t>(m0 + m) * n + row;
            float sum = acc[m];
            if (epilogue == EPILOGUE_RESIDUAL_F32) sum = bf16_bits_to_f32(residual[index]) + sum;
            else if (epilogue == EPILOGUE_RESIDUAL_ROUNDED) sum = round_bf16(sum) + bf16_bits_to_f32(residual[index]);
            y[index] = static_cast<uint16_t>(f32_to_bf16_bits(sum));
        }
}

cudaError_t launch_linear_fp8(const uint8_t *xq, const float *xscale, const uint8_t *w, const uint16_t *wscale,
                              uint16_t *y, const uint16_t *residual, int lanes, int n, int k, int epilogue,
                              cudaStream_t stream) {
    if (lanes <= 0) return cudaSuccess;
    if (k % 128 != 0) return cudaErrorInvalidValue;
    dim3 grid((n + 7) / 8, (lanes + 7) / 8);
    linear_fp8_kernel<8><<<grid, 256, 0, stream>>>(xq, xscale, w, wscale, y, residual, lanes, n, k, epilogue);
    return cudaGetLastError();
}

template <int MT>
__global__ void __launch_bounds__(256)
linear_silu_multiply_fp8_kernel(const uint8_t *__restrict__ xq, const float *__restrict__ xscale,
                                const uint8_t *__restrict__ wg, const uint16_t *__restrict__ wg_scale,
                                const uint8_t *__restrict__ wu, const uint16_t *__restrict__ wu_scale,
                                uint16_t *__restrict__ y, int lanes, int n, int k) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * 8 + warp;
    const int m0 = blockIdx.y * MT;
    if (row >= n) return;
    float gate[MT], up[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) gate[m] = up[m] = 0.0f;
    grid_dependency_wait();
    fp8_row_dot<MT>(xq, xscale, wg + static_cast<size_t>(row) * k, wg_scale + static_cast<size_t>(row >> 7) * (k >> 7), k,
                    lanes, m0, lane, gate);
    fp8_row_dot<MT>(xq, xscale, wu + static_cast<size_t>(row) * k, wu_scale + static_cast<size_t>(row >> 7) * (k >> 7), k,
                    lanes, m0, lane, up);
#pragma unroll
    for (int m = 0; m < MT; m++) {
        gate[m] = warp_sum(gate[m]);
        up[m] = warp_sum(up[m]);
    }
    if (lane == 0)
#pragma unroll
        for (int m = 0; m < MT; m++) {
            if (m0 + m >= lanes) break;
            float value = rounded_silu(round_bf16(gate[m])) * round_bf16(up[m]);
            y[static_cast<size_t>(m0 + m) * n + row] = static_cast<uint16_t>(f32_to_bf16_bits(value));
        }
}

cudaError_t launch_linear_silu_multiply_fp8(const uint8_t *xq, const float *xscale, const uint8_t *wg,
                                            const uint16_t *wg_scale, const uint8_t *wu, const uint16_t *wu_scale,
                                            uint16_t *y, int lanes, int n, int k, cudaStream_t stream) {
    if (lanes <= 0) return cudaSuccess;
    if (k % 128 != 0) return cudaErrorInvalidValue;
    dim3 grid((n + 7) / 8, (lanes + 7) / 8);
    linear_silu_multiply_fp8_kernel<8><<<grid, 256, 0, stream>>>(xq, xscale, wg, wg_scale, wu, wu_scale, y, lanes, n, k);
    return cudaGetLastError();
}

// ----------------------------------------------------------------------------- MoE experts (FP8)

// sparse_moe_gate_up_fp8_e4m3.comp.template:94-198.  grid = (ceil(inter/8), top_k, lanes); each CTA quantises the
// lane's hidden frame per 128 columns into shared memory (as the shader does), then one warp per intermediate row
// computes gate and up of the routed expert.  Experts outside [expert_start, expert_start+expert_count) are skipped
// (expert-parallel shards); their slot of `intermediates` is left untouched.
__global__ void __launch_bounds__(256)
moe_gate_up_fp8_kernel(const uint16_t *__restrict__ hidden, const uint32_t *__restrict__ routes,
                       const uint8_t *__restrict__ w, const uint16_t *__restrict__ wscale,
                       uint16_t *__restrict__ intermediates, int hidden_size, int inter, int experts, int top_k,
                       int expert_start, int expert_count) {
    extern __shared__ uint8_t shared[];
    const int token = blockIdx.z, route = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int blocks = hidden_size >> 7;
    uint8_t *hq = shared;
    float *hs = reinterpret_cast<float *>(shared + hidden_size);
    grid_dependency_wait();
    uint32_t packed_route = routes[static_cast<size_t>(token) * top_k + route];
    int expert = static_cast<int>(packed_route & 0xffffu);
    if (expert >= experts || expert < expert_start || expert >= expert_start + expert_count) return;
    expert -= expert_start;
    for (int block = warp; block < blocks; block += 8) {
        const uint32_t *src = reinterpret_cast<const uint32_t *>(hidden + static_cast<size_t>(token) * hidden_size + block * 128) + lane * 2;
        uint32_t w0 = src[0], w1 = src[1];
        float v0 = bf16_lo(w0), v1 = bf16_hi(w0), v2 = bf16_lo(w1), v3 = bf16_hi(w1);
        float block_max = warp_max(fmaxf(fmaxf(fabsf(v0), fabsf(v1)), fmaxf(fabsf(v2), fabsf(v3))));
        float scale = block_max > 0.0f ? block_max / 448.0f : 1.0f;
        if (lane == 0) hs[block] = scale;
        uint32_t q = static_cast<uint32_t>(f32_to_e4m3(v0 / scale)) | (static_cast<uint32_t>(f32_to_e4m3(v1 / scale)) << 8) |
                     (static_cast<uint32_t>(f32_to_e4m3(v2 / scale)) << 16) | (static_cast<uint32_t>(f32_to_e4m3(v3 / scale)) << 24);
        reinterpret_cast<uint32_t *>(hq + block * 128)[lane] = q;
    }
    __syncthreads();
    const int row = blockIdx.x * 8 + warp;
    if (row >= inter) return;
    const int scale_rows = (2 * inter + 127) >> 7;
    const uint8_t *wbase = w + static_cast<size_t>(expert) * 2 * inter * hidden_size;
    const uint16_t *sbase = wscale + static_cast<size_t>(expert) * scale_rows * blocks;
    float gate = 0.0f, up = 0.0f;
    for (int block = 0; block < blocks; block++) {
        uint32_t xq = reinterpret_cast<const uint32_t *>(hq + block * 128)[lane];
        float xf[4] = {e4m3_to_f32(xq & 0xff), e4m3_to_f32((xq >> 8) & 0xff), e4m3_to_f32((xq >> 16) & 0xff), e4m3_to_f32(xq >> 24)};
        uint32_t gq = __ldg(reinterpret_cast<const uint32_t *>(wbase + static_cast<size_t>(row) * hidden_size + block * 128) + lane);
        uint32_t uq = __ldg(reinterpret_cast<const uint32_t *>(wbase + static_cast<size_t>(inter + row) * hidden_size + block * 128) + lane);
        float gd = xf[0] * e4m3_to_f32(gq & 0xff) + xf[1] * e4m3_to_f32((gq >> 8) & 0xff) + xf[2] * e4m3_to_f32((gq >> 16) & 0xff) +
                   xf[3] * e4m3_to_f32(gq >> 24);
        float ud = xf[0] * e4m3_to_f32(uq & 0xff) + xf[1] * e4m3_to_f32((uq >> 8) & 0xff) + xf[2] * e4m3_to_f32((uq >> 16) & 0xff) +
                   xf[3] * e4m3_to_f32(uq >> 24);
        gate = fmaf(gd, hs[block] * bf16_bits_to_f32(sbase[static_cast<size_t>(row >> 7) * blocks + block]), gate);
        up = fmaf(ud, hs[block] * bf16_bits_to_f32(sbase[static_cast<size_t>((inter + row) >> 7) * blocks + block]), up);
    }
    gate = warp_sum(gate);
    up = warp_sum(up);
    if (lane == 0) {
        gate = round_bf16(gate);
        up = round_bf16(up);
        float value = round_bf16(round_bf16(gate / (1.0f + expf(-gate))) * up);
        intermediates[(static_cast<size_t>(token) * top_k + route) * inter + row] = static_cast<uint16_t>(f32_to_bf16_bits(value));
    }
}

cudaError_t launch_moe_gate_up_fp8(const uint16_t *hidden, const uint32_t *routes, const uint8_t *w,
                                   const uint16_t *wscale, uint16_t *intermediates, int lanes, int hidden_size,
                                   int inter, int experts, int top_k, int expert_start, int expert_count,
                                   cudaStream_t stream) {
    if (lanes <= 0) return cudaSuccess;
    if (hidden_size % 128 != 0) return cudaErrorInvalidValue;
    dim3 grid((inter + 7) / 8, top_k, lanes);
    size_t shared = hidden_size + sizeof(float) * (hidden_size / 128);
    moe_gate_up_fp8_kernel<<<grid, 256, shared, stream>>>(hidden, routes, w, wscale, intermediates, hidden_size, inter,
                                                          experts, top_k, expert_start, expert_count);
    return cudaGetLastError();
}

// sparse_moe_down_fp8_e4m3.comp.template:90-176: out = bf16(bf16(sum) * route_weight)
__global__ void __launch_bounds__(256)
moe_down_fp8_kernel(const uint16_t *__restrict__ intermediates, const uint32_t *__restrict__ routes,
                    const uint8_t *__restrict__ w, const uint16_t *__restrict__ wscale, uint16_t *__restrict__ outputs,
                    int hidden_size, int inter, int experts, int top_k, int expert_start, int expert_count) {
    extern __shared__ uint8_t shared[];
    const int token = blockIdx.z, route = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int blocks = inter >> 7;
    uint8_t *mq = shared;
    float *ms = reinterpret_cast<float *>(shared + inter);
    grid_dependency_wait();
    uint32_t packed_route = routes[static_cast<size_t>(token) * top_k + route];
    int expert = static_cast<int>(packed_route & 0xffffu);
    if (expert >= experts || expert < expert_start || expert >= expert_start + expert_count) return;
    expert -= expert_start;
    float route_weight = bf16_bits_to_f32(packed_route >> 16);
    const uint16_t *mid = intermediates + (static_cast<size_t>(token) * top_k + route) * inter;
    for (int block = warp; block < blocks; block += 8) {
        const uint32_t *src = reinterpret_cast<const uint32_t *>(mid + block * 128) + lane * 2;
        uint32_t w0 = src[0], w1 = src[1];
        float v0 = bf16_lo(w0), v1 = bf16_hi(w0), v2 = bf16_lo(w1), v3 = bf16_hi(w1);
        float block_max = warp_max(fmaxf(fmaxf(fabsf(v0), fabsf(v1)), fmaxf(fabsf(v2), fabsf(v3))));
        float scale = block_max > 0.0f ? block_max / 448.0f : 1.0f;
        if (lane == 0) ms[block] = scale;
        uint32_t q = static_cast<uint32_t>(f32_to_e4m3(v0 / scale)) | (static_cast<uint32_t>(f32_to_e4m3(v1 / scale)) << 8) |
                     (static_cast<uint32_t>(f32_to_e4m3(v2 / scale)) << 16) | (static_cast<uint32_t>(f32_to_e4m3(v3 / scale)) << 24);
        reinterpret_cast<uint32_t *>(mq + block * 128)[lane] = q;
    }
    __syncthreads();
    const int row = blockIdx.x * 8 + warp;
    if (row >= hidden_size) return;
    const int scale_rows = (hidden_size + 127) >> 7;
    const uint8_t *wbase = w + static_cast<size_t>(expert) * hidden_size * inter;
    const uint16_t *sbase = wscale + static_cast<size_t>(expert) * scale_rows * blocks;
    float sum = 0.0f;
    for (int block = 0; block < blocks; block++) {
        uint32_t xq = reinterpret_cast<const uint32_t *>(mq + block * 128)[lane];
        uint32_t wq = __ldg(reinterpret_cast<const uint32_t *>(wbase + static_cast<size_t>(row) * inter + block * 128) + lane);
        float d = e4m3_to_f32(xq & 0xff) * e4m3_to_f32(wq & 0xff) + e4m3_to_f32((xq >> 8) & 0xff) * e4m3_to_f32((wq >> 8) & 0xff) +
                  e4m3_to_f32((xq >> 16) & 0xff) * e4m3_to_f32((wq >> 16) & 0xff) + e4m3_to_f32(xq >> 24) * e4m3_to_f32(wq >> 24);
        sum = fmaf(d, ms[block] * bf16_bits_to_f32(sbase[static_cast<size_t>(row >> 7) * blocks + block]), sum);
    }
    sum = warp_sum(sum);
    if (lane == 0)
        outputs[(static_cast<size_t>(token) * top_k + route) * hidden_size + row] =
            static_cast<uint16_t>(f32_to_bf16_bits(round_bf16(sum) * route_weight));
}

cudaError_t launch_moe_down_fp8(const uint16_t *intermediates, const uint32_t *routes, const uint8_t *w,
                                const uint16_t *wscale, uint16_t *outputs, int lanes, int hidden_size, int inter,
                                int experts, int top_k, int expert_start, int expert_count, cudaStream_t stream) {
    if (lanes <= 0) return cudaSuccess;
    if (inter % 128 != 0) return cudaErrorInvalidValue;
    dim3 grid((hidden_size + 7) / 8, top_k, lanes);
    size_t shared = inter + sizeof(float) * (inter / 128);
    moe_down_fp8_kernel<<<grid, 256, shared, stream>>>(intermediates, routes, w, wscale, outputs, hidden_size, inter,
                                                       experts, top_k, expert_start, expert_count);
    return cudaGetLastError();
}

}  // namespace nerve

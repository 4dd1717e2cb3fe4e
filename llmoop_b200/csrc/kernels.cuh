// Launchers for the sm_100a kernels of the MTP decode path.  Activations are
// bf16 row-major [lane][width]; `lanes` is the batch of (stream, tick) pairs
// processed in one launch (verify candidates, prefill chunk, or multi-stream
// decode).  All functions enqueue on `stream` and return the launch status.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace nerve {

// Per-launch description of the lanes that touch transient state.
struct LaneTable {
    const uint32_t *position;  // [lanes] stream tick (low 32 bits) of each lane
    const int32_t *slot;       // [lanes] stream slot of each lane (row of block_table)
};

// Paged KV state of one attention layer.  Page p holds `page_tokens` tokens:
//   K at kv + p*page_elems + (head*page_tokens + t)*head_width
//   V at the same offset + page_elems/2
// A stream's logical token index i lives in page block_table[slot][ (i / page_tokens) % pages_per_slot ].
struct KvLayer {
    uint16_t *pool;
    const int32_t *block_table;  // [slots][pages_per_slot]
    int pages_per_slot;
    int page_tokens;
    int kv_heads;
    int head_width;
    uint32_t capacity;  // pages_per_slot * page_tokens (ring length in tokens)
};

cudaError_t launch_embedding(const uint16_t *table, const uint32_t *tokens, uint16_t *out, int lanes, int width,
                             int vocab, float scale, cudaStream_t stream);

cudaError_t launch_rms_norm(const uint16_t *x, const uint16_t *weight, uint16_t *y, int lanes, int width, float eps,
                            float weight_offset, cudaStream_t stream);

cudaError_t launch_add(const uint16_t *a, const uint16_t *b, uint16_t *y, size_t count, cudaStream_t stream);
cudaError_t launch_silu_multiply(const uint16_t *gate, const uint16_t *up, uint16_t *y, size_t count, cudaStream_t stream);
cudaError_t launch_concat(const uint16_t *a, const uint16_t *b, uint16_t *y, int lanes, int width_a, int width_b,
                          cudaStream_t stream);

// RoPE from a host-built table: cos_sin[(position % table_positions) * rotary/2 + f] = {bf16 cos, bf16 sin} packed
// in one u32 (cos low).  Optional per-head RMSNorm first (norm_weight != nullptr).
cudaError_t launch_rope(const uint16_t *x, uint16_t *y, const uint32_t *cos_sin, uint32_t table_positions,
                        const uint32_t *positions, int lanes, int heads, int head_width, int rotary, int interleaved,
                        const uint16_t *norm_weight, float eps, float weight_offset, cudaStream_t stream);

enum LinearEpilogue {
    EPILOGUE_BF16 = 0,            // y = bf16(sum)
    EPILOGUE_RESIDUAL_ROUNDED = 1,  // y = bf16(bf16(sum) + residual)        (BF16 / INT4 packages)
    EPILOGUE_RESIDUAL_F32 = 2,    // y = bf16(sum + residual)                (FP8 packages)
    EPILOGUE_F32_SCALED = 3,      // y_f32 = sum * scale                     (logits; tensor-parallel partial sums)
};

// y[m][n] = sum_k x[m][k] * W[n][k], bf16 weights.
cudaError_t launch_linear_bf16(const uint16_t *x, const uint16_t *w, void *y, const uint16_t *residual, int lanes,
                               int n, int k, int epilogue, float scale, cudaStream_t stream, int *error_flag = nullptr);
// y = bf16( silu_bf16(bf16(x.Wg)) * bf16(x.Wu) )
cudaError_t launch_linear_silu_multiply_bf16(const uint16_t *x, const uint16_t *wg, const uint16_t *wu, uint16_t *y,
                                             int lanes, int n, int k, cudaStream_t stream);

// INT4 compressed-tensors weight-only linear: qweight [n][k/8] u32, scales bf16 [n][k/group].
// error_flag (optional device word): set to 3 by the wide-batch GEMM if one of its bounded waits expires.
cudaError_t launch_linear_int4(const uint16_t *x, const uint32_t *qweight, const uint16_t *scales, uint16_t *y,
                               const uint16_t *residual, int lanes, int n, int k, int group, int epilogue,
                               cudaStream_t stream, int *error_flag = nullptr);

// FP8 W8A8: xq e4m3 [lanes][k], xscale f32 [lanes][k/128]; w e4m3 [n][k]; wscale bf16 [ceil(n/128)][k/128].
cudaError_t launch_quantize_fp8(const uint16_t *x, uint8_t *q, float *scales, int lanes, int k, cudaStream_t stream);
cudaError_t launch_linear_fp8(const uint8_t *xq, const float *xscale, const uint8_t *w, const uint16_t *wscale,
                              uint16_t *y, const uint16_t *residual, int lanes, int n, int k, int epilogue,
                              cudaStream_t stream);
cudaError_t launch_linear_silu_multiply_fp8(const uint8_t *xq, const float *xscale, const uint8_t *wg,
                                            const uint16_t *wg_scale, const uint8_t *wu, const uint16_t *wu_scale,
                                            uint16_t *y, int lanes, int n, int k, cudaStream_t stream);

// MoE (softmax over the selected experts, routes sorted by expert id).
cudaError_t launch_moe_topk(const uint16_t *router_logits, uint32_t *routes, int lanes, int experts, int top_k,
                            cudaStream_t stream);
cudaError_t launch_moe_gate_up_fp8(const uint16_t *hidden, const uint32_t *routes, const uint8_t *w,
                                   const uint16_t *wscale, uint16_t *intermediates, int lanes, int hidden_size,
                                   int inter, int experts, int top_k, int expert_start, int expert_count,
                                   cudaStream_t stream);
cudaError_t launch_moe_down_fp8(const uint16_t *intermediates, const uint32_t *routes, const uint8_t *w,
                                const uint16_t *wscale, uint16_t *outputs, int lanes, int hidden_size, int inter,
                                int experts, int top_k, int expert_start, int expert_count, cudaStream_t stream);
cudaError_t launch_moe_reduce(const uint16_t *outputs, uint16_t *y, int lanes, int hidden_size, int top_k,
                              float routed_scale, cudaStream_t stream);

// Append K,V of every lane at its position, then causal GQA attention over the
// stream's pages: split over the context, partials merged by a second kernel.
// scratch holds [lanes][q_heads][splits][head_width + 2] f32.
size_t attention_scratch_bytes(int lanes, int q_heads, int head_width, int max_splits);
cudaError_t launch_kv_append(const uint16_t *k, const uint16_t *v, const KvLayer &kv, const LaneTable &lanes_meta,
                             int lanes, cudaStream_t stream);
// Lanes are stream-major: every stream of the batch contributes `lanes_per_stream` consecutive lanes.
cudaError_t launch_attention(const uint16_t *q, uint16_t *out, const KvLayer &kv, const LaneTable &lanes_meta,
                             int lanes, int lanes_per_stream, int q_heads, float scale, int split_tokens, int max_splits,
                             float *scratch, cudaStream_t stream);

// INT4 multi-branch forms (one launch for q/k/v; gate/up with the SiLU*up epilogue).
cudaError_t launch_linear_int4_multi(const uint16_t *x, int branches, const uint32_t *const *qweights,
                                     const uint16_t *const *scales, uint16_t *const *ys, const int *ns,
                                     const uint16_t *residual, int lanes, int k, int epilogue, cudaStream_t stream,
                                     int *error_flag = nullptr);
cudaError_t launch_linear_int4_silu_pair(const uint16_t *x, const uint32_t *gate_q, const uint16_t *gate_s,
                                         const uint32_t *up_q, const uint16_t *up_s, uint16_t *y, int lanes, int n,
                                         int k, cudaStream_t stream);

// ---- streaming output projection for at most 8 lanes (kernels_projection.cu) ----
// logits[lane][row] = scale * x[lane] . table[first_row + row], f32, rows of a slice that starts at a multiple of 16.
// `streamed_table` is the copy launch_projection_table makes of the whole bf16 table (projection_table_bytes bytes).
// With `rounded` set the kernel is a plain bf16 linear instead: rounded[lane][row] = bf16(sum), `logits` and `scale` unused.
size_t projection_table_bytes(int rows, int k);
cudaError_t launch_projection_table(const uint16_t *table, void *out, int rows, int k, cudaStream_t stream);
bool output_projection_supported(int lanes, int k);
cudaError_t launch_output_projection(const uint16_t *x, const void *streamed_table, int first_row, float *logits, int lanes, int rows, int k, float scale,
                                     int grid, int *error_flag, cudaStream_t stream, uint16_t *rounded = nullptr);

// ---- INT4 g128 GEMM on the tcgen05 tensor cores for 64 lanes and more (kernels_int4_gemm.cu) ----
// One CTA per 128 rows x 64 lanes; the launchers above use it for such batches.  y and the epilogues as for
// launch_linear_int4 (EPILOGUE_F32_SCALED writes f32 * scale).  error_flag (optional device word) is set to 3 if a
// bounded wait for the tensor core expires.
bool linear_int4_gemm_supported(int lanes, int n, int k);
// bf16 weights, batches of 16 lanes and more (tcgen05): called by launch_linear_bf16.
bool linear_bf16_gemm_supported(int lanes, int n, int k);
cudaError_t launch_linear_bf16_gemm(const uint16_t *x, const uint16_t *w, void *y, const uint16_t *residual, int lanes, int n, int k, int epilogue,
                                    float scale, int *error_flag, cudaStream_t stream);
cudaError_t launch_linear_int4_gemm_multi(const uint16_t *x, int branches, const uint32_t *const *qweights, const uint16_t *const *scales, void *const *ys,
                                          const int *ns, const uint16_t *residual, int lanes, int k, int epilogue, float scale, int *error_flag,
                                          cudaStream_t stream);
cudaError_t launch_linear_int4_gemm(const uint16_t *x, const uint32_t *qweight, const uint16_t *scales, void *y, const uint16_t *residual, int lanes,
                                    int n, int k, int epilogue, float scale, int *error_flag, cudaStream_t stream);

// ---- persistent decode stack (kernels_stack.cu) ----
// One cooperative launch runs a whole stack of dense INT4 g128 Llama-style layers for a batch of at most 8 lanes:
// every CTA (one per SM) streams its share of each weight matrix while grid-wide barriers separate the steps of a
// layer.  Weights are read from per-CTA byte streams written at mount (launch_int4_cta_streams).

// How the CTAs of a grid share one matrix of `tiles` 16-row tiles (a gate/up pair tile holds 16 gate rows and the
// same 16 up rows: rt = 2) over K = groups * 128 columns.  CTA c owns tiles c, c + grid, ...; it works on `slots`
// of them at a time (one pass), `width` warps per tile, warp i of a tile taking units i, i + width, ... of the
// tile's `units` = groups * rt blocks of 16x128 nibbles (unit u = group u / rt, matrix u % rt).  Step s of a pass
// is one stage of the CTA's stream: for every present tile slot, units s * width .. s * width + width - 1
// (1 KB of nibbles each, zero beyond `units`), followed by the same units' 32-byte scale-pair rows.
struct MatrixSchedule {
    int tiles, units, rt, slots, width, steps, grid;
};
__host__ __device__ inline MatrixSchedule stack_schedule(int tiles, int groups, int rt, int grid) {
    MatrixSchedule s;
    s.tiles = tiles;
    s.rt = rt;
    s.units = groups * rt;
    s.grid = grid;
    const int most = (tiles + grid - 1) / grid;
    int slots = 1;
    while (slots < most && slots * 2 <= 16 / rt) slots *= 2;
    int width = 16 / slots;
    while (width / 2 >= rt && width / 2 >= s.units) width /= 2;
    s.slots = slots;
    s.width = width;
    s.steps = (s.units + width - 1) / width;
    return s;
}
__host__ __device__ inline int stack_cta_tiles(const MatrixSchedule &s, int cta) { return s.tiles / s.grid + (cta < s.tiles % s.grid ? 1 : 0); }
// Bytes of the stream in front of CTA `cta`'s share (every tile costs width * steps units of 1056 bytes).
__host__ __device__ inline size_t stack_cta_offset(const MatrixSchedule &s, int cta) {
    const int extra = s.tiles % s.grid;
    const size_t tiles_before = static_cast<size_t>(cta) * (s.tiles / s.grid) + (cta < extra ? cta : extra);
    return tiles_before * s.width * s.steps * 1056;
}
__host__ __device__ inline size_t stack_stream_bytes(const MatrixSchedule &s) { return static_cast<size_t>(s.tiles) * s.width * s.steps * 1056; }

struct StackLayer {
    const uint8_t *qkv, *o, *gate_up, *down;  // per-CTA streams of the four matrix steps
    const uint16_t *input_norm, *post_norm;
    KvLayer kv;
};
struct StackShape {
    int hidden, q_heads, kv_heads, head_width, ffn;
    float eps, norm_offset, attention_scale;
    const uint32_t *rope_table;  // [position][head_width / 2] packed (sin << 16 | cos) bf16
    uint32_t rope_positions;
    int grid;                    // CTAs the streams were written for (the device's SM count at mount)
};
struct StackBuffers {
    uint16_t *hidden;            // [lanes][hidden] residual stream, updated in place
    uint16_t *q;                 // [lanes][q_heads * head_width]
    float *attention_scratch;    // split partials, attention_scratch_bytes()
    uint16_t *attention_out;     // [lanes][q_heads * head_width] fp16 in fragment order (see kernels_stack.cu)
    uint16_t *activation;        // [lanes][ffn] fp16 in fragment order
    unsigned int *barrier;       // STACK_BARRIER_WORDS words, zero before the first launch
    int *error_flag;             // set when a bounded wait expires (2: grid barrier or peer, 3: weight pipeline)
    unsigned long long *timing;  // optional [layers][32] nanosecond stamps of CTA 0 (step boundaries), or nullptr
    unsigned int barrier_handicap;  // test hook: arrivals the grid barriers wait for on top of the grid's own (0 in service);
                                    // they can never come, so the first barrier gives up after a short bounded wait
};
constexpr int STACK_BARRIER_WORDS = 1024;  // two barrier words, then the attention arrival counters (kv heads x lane groups)
// Tensor-parallel exchange of the persistent kernel: every rank holds the same residual stream and its shard of
// each layer.  The o and down projections push their f32 partial sums into every peer's inbox - value and exchange
// number in one 8-byte store over NVLink - and the thread that owns an output element waits for the peers' words
// in its own rank's inbox, then adds all shares in rank order.
// Inbox of a rank: [2 parities][STACK_TP_MAX_RANKS sources][8 lanes][hidden] 8-byte words.
constexpr int STACK_TP_MAX_RANKS = 8;
constexpr int STACK_TP_WORD_CONSUMED = 2;                // control word: exchanges done by earlier launches
constexpr unsigned int STACK_TP_SPIN_LIMIT = 1u << 25;   // polls of one inbox word: ranks start their launches a host jitter apart
struct StackTp {
    int rank = 0, size = 1;                            // size 1: no exchange
    float *exchange[STACK_TP_MAX_RANKS] = {};          // every rank's inbox as seen from this GPU (own entry: local memory)
    unsigned long long *counter[STACK_TP_MAX_RANKS] = {};  // every rank's 16 control words
};
constexpr int STACK_TP_WORD_VOTES = 3;                   // control word: arg-max votes taken so far (tensor_parallel_argmax)
constexpr int STACK_TP_VOTE_LANES = 64;                  // lanes one vote can carry
// Behind the 16 control words: the vote area [2 parities][STACK_TP_MAX_RANKS][STACK_TP_VOTE_LANES][2] 8-byte words.
constexpr size_t STACK_TP_CONTROL_BYTES = 16 * sizeof(unsigned long long) + 2 * STACK_TP_MAX_RANKS * STACK_TP_VOTE_LANES * 2 * sizeof(unsigned long long);
inline size_t stack_tp_exchange_floats(int hidden) { return static_cast<size_t>(2) * STACK_TP_MAX_RANKS * 8 * hidden * 2; }

// One source matrix of a stream copy.  rope_head_width > 0 orders the rows of every head so that MMA rows
// r and r + 8 of a tile are the rotary partners (d, d + head_width / 2).
struct RelayoutSegment {
    const uint32_t *qweight;
    const uint16_t *scales;
    int rows;
    int rope_head_width;
};
// Segments share K; their tiles follow one another, or - with `pair` - segment 0 and 1 are interleaved unit by unit
// (gate, up).  Every segment's row count must be a multiple of 16.  `rows` of int4_cta_stream_bytes is the sum of
// the segments' rows (one segment's for a pair).
size_t int4_cta_stream_bytes(int rows, int k, bool pair, int grid);
cudaError_t launch_int4_cta_streams(const RelayoutSegment *segments, int count, bool pair, int k, int grid, uint8_t *out,
                                    cudaStream_t stream);
// Whether the stack kernel is built for this shape and batch; *smem_bytes receives its dynamic shared memory.
bool decode_stack_supported(const StackShape &shape, int lanes, size_t *smem_bytes);
cudaError_t launch_decode_stack(const StackLayer *layers_device, int layer_count, const StackShape &shape,
                                const StackBuffers &buffers, const LaneTable &lanes_meta, int lanes, int lanes_per_stream,
                                int split_tokens, int max_splits, cudaStream_t stream, const StackTp *tp_device = nullptr, int tp_size = 1);

// Tensor-parallel row-parallel linears: out = bf16(bf16(sum) + residual) (or bf16(sum) without residual) from the
// all-reduced f32 sums [count].
cudaError_t launch_round_add(const float *sums, const uint16_t *residual, uint16_t *out, size_t count, cudaStream_t stream);

// ---- glue of the speculative cycle (all tiny) ----
// dst[i] = src[index[i]] for rows of `width` bf16.
cudaError_t launch_gather_rows(const uint16_t *src, const int32_t *index, uint16_t *dst, int rows, int width,
                               cudaStream_t stream);
// Hidden inputs of the draft catch-up: lane (s, 0) takes pending[slot[s]], lane (s, i>0) takes normalized (s, i-1).
cudaError_t launch_shift_hidden(const uint16_t *pending, const int32_t *slots, const uint16_t *normalized,
                                uint16_t *dst, int streams, int lanes_per_stream, int hidden, cudaStream_t stream);
// After draft step `step`: token = forced[s][step] unless it is 0xffffffff, else the sampled record; written to
// next_tokens[s] and verify_tokens[s][step + 1].
cudaError_t launch_draft_select(const uint32_t *records, const uint32_t *forced, int step, int streams, int drafts,
                                uint32_t *next_tokens, uint32_t *verify_tokens, cudaStream_t stream);
// Longest-matching-prefix acceptance + stop truncation (speculative_decode.rs:54-105) per stream, then
// pending[slot[s]] = normalized lane (s, committed-1).  out row = {accepted, committed, emitted_count, 0,
// emitted[drafts+1], targets[drafts+1]}.
cudaError_t launch_accept(const uint32_t *verify_tokens, const uint32_t *target_records, const uint32_t *stop_tokens,
                          const int32_t *stop_counts, int max_stop, int streams, int drafts, uint32_t *out,
                          const uint16_t *normalized, uint16_t *pending, const int32_t *slots, int hidden,
                          cudaStream_t stream);

// Vocabulary-parallel greedy sampling under tensor parallelism: every rank has taken the arg-max of its own slice of
// the vocabulary (records_local: {token within the slice, logit bits, ..} per lane, as launch_argmax writes them);
// the ranks push (logit, global token), tagged with the vote number, into each other's vote areas over NVLink, wait
// (bounded) for all of them and all pick the same winner - highest logit, ties to the lowest token id.  One block.
// The vote number lives on the device (control word STACK_TP_WORD_VOTES), so the launch can be replayed from a graph.
cudaError_t launch_tensor_parallel_argmax(const uint32_t *records_local, uint32_t first_token, uint32_t *records, int lanes, const StackTp *tp_device,
                                          int *error_flag, cudaStream_t stream);

// Greedy arg-max (ties -> lowest id); record = {token, logit bits, 0, 0} per lane.
// `scratch` holds argmax_scratch_bytes(lanes) bytes of per-chunk partial winners.
size_t argmax_scratch_bytes(int lanes);
cudaError_t launch_argmax(const float *logits, uint32_t *records, int lanes, int vocab, void *scratch, cudaStream_t stream);
// The same with the partial winners in a fixed device array of the library (no allocation anywhere); at most
// argmax_static_max_lanes() lanes, one call at a time per device.
int argmax_static_max_lanes();
cudaError_t launch_argmax_static(const float *logits, uint32_t *records, int lanes, int vocab, cudaStream_t stream);

// ---- seeded temperature / top-k / top-p / min-p sampler (kernels_sampler.cu) ----
constexpr int SAMPLER_MAX_TOP_K = 64;
struct SamplerParams {   // one per stream slot
    uint32_t method;     // 0 greedy (arg-max, record flags 0), 1 temperature_top_k_top_p
    uint32_t top_k;      // 1..SAMPLER_MAX_TOP_K
    uint32_t seed;
    float temperature, top_p, min_p;
};
size_t sampler_scratch_bytes(int lanes);
// One record {token, logit bits, sampled flag, 0} per lane; lane l uses table[slots[l]] (slot 0 when slots is
// NULL) and the uniform of stream tick ticks[l].
cudaError_t launch_sample(const float *logits, uint32_t *records, int lanes, int vocab, const SamplerParams *table, const int32_t *slots,
                          const uint32_t *ticks, void *scratch, cudaStream_t stream);

}  // namespace nerve

// Glue kernels of the speculative cycle: everything the reference does on the
// host between submits (token hand-over between draft steps, prefix
// acceptance, stop truncation, pending-hidden bookkeeping) runs on the device
// so that one cycle is a single stream of launches with one host read-back.
#include "common.cuh"
#include "kernels.cuh"

namespace nerve {

__global__ void gather_rows_kernel(const uint32_t *__restrict__ src, const int32_t *__restrict__ index,
                                   uint32_t *__restrict__ dst, int words) {
    grid_dependency_wait();
    int row = blockIdx.x;
    int source = index[row];
    if (source < 0) return;
    for (int word = threadIdx.x; word < words; word += blockDim.x)
        dst[static_cast<size_t>(row) * words + word] = src[static_cast<size_t>(source) * words + word];
}

cudaError_t launch_gather_rows(const uint16_t *src, const int32_t *index, uint16_t *dst, int rows, int width,
                               cudaStream_t stream) {
    if (rows <= 0) return cudaSuccess;
    gather_rows_kernel<<<rows, 256, 0, stream>>>(reinterpret_cast<const uint32_t *>(src), index,
                                                 reinterpret_cast<uint32_t *>(dst), width / 2);
    return cudaGetLastError();
}

__global__ void shift_hidden_kernel(const uint32_t *__restrict__ pending, const int32_t *__restrict__ slots,
                                    const uint32_t *__restrict__ normalized, uint32_t *__restrict__ dst,
                                    int lanes_per_stream, int words) {
    grid_dependency_wait();
    int lane = blockIdx.x;
    int s = lane / lanes_per_stream, i = lane % lanes_per_stream;
    const uint32_t *source = i == 0 ? pending + static_cast<size_t>(slots[s]) * words
                                    : normalized + static_cast<size_t>(lane - 1) * words;
    for (int word = threadIdx.x; word < words; word += blockDim.x) dst[static_cast<size_t>(lane) * words + word] = source[word];
}

cudaError_t launch_shift_hidden(const uint16_t *pending, const int32_t *slots, const uint16_t *normalized,
                                uint16_t *dst, int streams, int lanes_per_stream, int hidden, cudaStream_t stream) {
    if (streams <= 0) return cudaSuccess;
    shift_hidden_kernel<<<streams * lanes_per_stream, 256, 0, stream>>>(
        reinterpret_cast<const uint32_t *>(pending), slots, reinterpret_cast<const uint32_t *>(normalized),
        reinterpret_cast<uint32_t *>(dst), lanes_per_stream, hidden / 2);
    return cudaGetLastError();
}

__global__ void draft_select_kernel(const uint32_t *__restrict__ records, const uint32_t *__restrict__ forced, int step,
                                    int streams, int drafts, uint32_t *__restrict__ next_tokens,
                                    uint32_t *__restrict__ verify_tokens) {
    grid_dependency_wait();
    int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= streams) return;
    uint32_t token = records[static_cast<size_t>(s) * 4];
    if (forced != nullptr) {
        uint32_t override_token = forced[static_cast<size_t>(s) * drafts + step];
        if (override_token != 0xffffffffu) token = override_token;
    }
    next_tokens[s] = token;
    verify_tokens[static_cast<size_t>(s) * (drafts + 1) + step + 1] = token;
}

cudaError_t launch_draft_select(const uint32_t *records, const uint32_t *forced, int step, int streams, int drafts,
                                uint32_t *next_tokens, uint32_t *verify_tokens, cudaStream_t stream) {
    if (streams <= 0) return cudaSuccess;
    draft_select_kernel<<<(streams + 63) / 64, 64, 0, stream>>>(records, forced, step, streams, drafts, next_tokens,
                                                                verify_tokens);
    return cudaGetLastError();
}

__global__ void accept_kernel(const uint32_t *__restrict__ verify_tokens, const uint32_t *__restrict__ target_records,
                              const uint32_t *__restrict__ stop_tokens, const int32_t *__restrict__ stop_counts,
                              int max_stop, int drafts, uint32_t *__restrict__ out, const uint32_t *__restrict__ normalized,
                              uint32_t *__restrict__ pending, const int32_t *__restrict__ slots, int words) {
    grid_dependency_wait();
    __shared__ int committed_shared;
    const int s = blockIdx.x;
    const int width = drafts + 1;
    uint32_t *row = out + static_cast<size_t>(s) * (4 + 2 * width);
    if (threadIdx.x == 0) {
        const uint32_t *inputs = verify_tokens + static_cast<size_t>(s) * width;  // [x, d_1 .. d_k]
        int accepted = 0;
        while (accepted < drafts && inputs[accepted + 1] == target_records[(static_cast<size_t>(s) * width + accepted) * 4]) accepted++;
        int committed = accepted + 1;
        int count = 0;
        for (int i = 0; i < accepted; i++) row[4 + count++] = inputs[i + 1];
        row[4 + count++] = target_records[(static_cast<size_t>(s) * width + accepted) * 4];
        const int stops = stop_counts[s];
        for (int i = 0; i < count; i++) {
            bool is_stop = false;
            for (int t = 0; t < stops; t++) is_stop |= stop_tokens[static_cast<size_t>(s) * max_stop + t] == row[4 + i];
            if (is_stop) {
                if (accepted > i + 1) accepted = i + 1;
                committed = i + 1;
                count = i + 1;
                break;
            }
        }
        row[0] = static_cast<uint32_t>(accepted);
        row[1] = static_cast<uint32_t>(committed);
        row[2] = static_cast<uint32_t>(count);
        row[3] = 0u;
        for (int i = 0; i < width; i++) row[4 + width + i] = target_records[(static_cast<size_t>(s) * width + i) * 4];
        committed_shared = committed;
    }
    __syncthreads();
    const uint32_t *source = normalized + (static_cast<size_t>(s) * width + committed_shared - 1) * words;
    uint32_t *destination = pending + static_cast<size_t>(slots[s]) * words;
    for (int word = threadIdx.x; word < words; word += blockDim.x) destination[word] = source[word];
}

cudaError_t launch_accept(const uint32_t *verify_tokens, const uint32_t *target_records, const uint32_t *stop_tokens,
                          const int32_t *stop_counts, int max_stop, int streams, int drafts, uint32_t *out,
                          const uint16_t *normalized, uint16_t *pending, const int32_t *slots, int hidden,
                          cudaStream_t stream) {
    if (streams <= 0) return cudaSuccess;
    accept_kernel<<<streams, 256, 0, stream>>>(verify_tokens, target_records, stop_tokens, stop_counts, max_stop, drafts,
                                               out, reinterpret_cast<const uint32_t *>(normalized),
                                               reinterpret_cast<uint32_t *>(pending), slots, hidden / 2);
    return cudaGetLastError();
}

// ---- vocabulary-parallel arg-max ------------------------------------------------------------------------------
// See launch_tensor_parallel_argmax in kernels.cuh.  Thread l serves lane l.  A vote word is (vote number << 32 |
// payload): the logit bits in the first word, the global token id in the second; a reader accepts a pair once both
// carry the number of the vote in progress.  Parities alternate per vote: a rank can only be one vote ahead of a
// peer (it needs the peer's word of vote v before it can finish v), so the slot of vote v + 2 is free by then.
__global__ void tensor_parallel_argmax_kernel(const uint32_t *__restrict__ records_local, uint32_t first_token, uint32_t *__restrict__ records,
                                              int lanes, const StackTp *__restrict__ tp_pointer, int *error_flag) {
    const StackTp &tp = *tp_pointer;
    unsigned long long *control = tp.counter[tp.rank];
    const uint32_t vote = static_cast<uint32_t>(control[STACK_TP_WORD_VOTES]) + 1u;  // every thread reads it before thread 0 moves it on (below)
    const int lane = threadIdx.x;
    const size_t parity_offset = static_cast<size_t>(vote & 1u) * STACK_TP_MAX_RANKS * STACK_TP_VOTE_LANES * 2;
    float best = 0.0f;
    uint32_t token = 0xffffffffu;
    if (lane < lanes) {
        const uint32_t local_token = records_local[lane * 4], logit_bits = records_local[lane * 4 + 1];
        const unsigned long long tag = static_cast<unsigned long long>(vote) << 32;
        for (int r = 0; r < tp.size; r++) {
            if (r == tp.rank) continue;
            unsigned long long *theirs = tp.counter[r] + 16 + parity_offset + (static_cast<size_t>(tp.rank) * STACK_TP_VOTE_LANES + lane) * 2;
            asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(theirs), "l"(tag | logit_bits) : "memory");
            asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(theirs + 1), "l"(tag | (local_token + first_token)) : "memory");
        }
        unsigned int spins = 0;
        bool gave_up = false;
        for (int r = 0; r < tp.size; r++) {
            float candidate = __uint_as_float(logit_bits);
            uint32_t candidate_token = local_token + first_token;
            if (r != tp.rank) {
                const unsigned long long *mine = control + 16 + parity_offset + (static_cast<size_t>(r) * STACK_TP_VOTE_LANES + lane) * 2;
                unsigned long long first = 0, second = 0;
                while (!gave_up) {
                    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(first) : "l"(mine) : "memory");
                    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(second) : "l"(mine + 1) : "memory");
                    if (static_cast<uint32_t>(first >> 32) == vote && static_cast<uint32_t>(second >> 32) == vote) break;
                    if (++spins > STACK_TP_SPIN_LIMIT) {
                        atomicExch(error_flag, 2);
                        gave_up = true;
                    } else if ((spins & 255u) == 0 && *reinterpret_cast<volatile int *>(error_flag) != 0) {
                        gave_up = true;
                    }
                }
                candidate = __uint_as_float(static_cast<uint32_t>(first));
                candidate_token = static_cast<uint32_t>(second);
            }
            if (token == 0xffffffffu || candidate > best || (candidate == best && candidate_token < token)) {
                best = candidate;
                token = candidate_token;
            }
        }
        uint32_t *record = records + static_cast<size_t>(lane) * 4;
        record[0] = token;
        record[1] = __float_as_uint(best);
        record[2] = 0u;
        record[3] = 0u;
    }
    __syncthreads();
    if (threadIdx.x == 0) control[STACK_TP_WORD_VOTES] = vote;
}

cudaError_t launch_tensor_parallel_argmax(const uint32_t *records_local, uint32_t first_token, uint32_t *records, int lanes, const StackTp *tp_device,
                                          int *error_flag, cudaStream_t stream) {
    if (lanes <= 0) return cudaSuccess;
    if (lanes > STACK_TP_VOTE_LANES || tp_device == nullptr) return cudaErrorInvalidValue;
    tensor_parallel_argmax_kernel<<<1, STACK_TP_VOTE_LANES, 0, stream>>>(records_local, first_token, records, lanes, tp_device, error_flag);
    return cudaGetLastError();
}

}  // namespace nerve

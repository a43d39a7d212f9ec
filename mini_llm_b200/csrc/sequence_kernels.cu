// Kernels of the mixers that are no softmax attention over keys and values per head, and of
// what stands around them: norms by root mean square in groups (also as the way a
// sublayer's result is added onto the residual stream, and with a sigmoid gate), a short
// causal convolution over time with its state, rotary positions in the interleaved layout,
// attention over a shared latent (all heads read one row per token; the row's first part is
// also the value), a batch of small products per head, the matrix-memory recurrence
// S <- a S + b k v^T with a fixed or a gated and stabilised decay, and the weighted sum of
// all layer results.
//
// Every kernel is templated on the element type of the activations (float: the true 32-bit
// path; bfloat16: the serving path).  Norm statistics, angles, scores, softmax, gates, decays
// and all recurrent state are 32-bit in both.  A step's entries are read from device arrays
// (slot, first row, rows, first position per entry), so a step of one shape launches the same
// kernels with the same arguments.  Every kernel is launched as a programmatic dependent of the
// kernel before it on its stream: its blocks may be scheduled while that one still runs, and the
// first thing each does is to wait for it, before any memory is touched.
#include "common.cuh"

MLLM_DEFINE_ERROR_API(mllm_sequence)

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float log_sigmoid_f(float z) {
    return z >= 0.0f ? -log1pf(expf(-z)) : z - log1pf(expf(z));
}

// ---------------------------------------------------------------------------
// Norm by root mean square in groups.  Row r of x (fp32) is cut into `groups` equal
// consecutive pieces; each is divided by sqrt(mean(piece^2) + eps); the whole is multiplied
// by the gain.  One block per (row, group).
//   ADD   out (fp32) += result            (a sublayer's result onto the residual stream)
//   GATE  1: result *= sigmoid(gate[r, c]); 2: result *= silu(gate[r, c]); 3: the INPUT is
//         multiplied by silu(gate[r, c]) before the root mean square is taken
//         (gate has the activations' element type)
// `rows` (may be null) gathers input rows.  out may be x itself.
// ---------------------------------------------------------------------------
template <typename O, typename G, bool ADD, int GATE>
__global__ void grouped_rms_norm_kernel(O* __restrict__ out, long ld_out, const float* x, long ld_x,
                                        const float* __restrict__ gain, const int* __restrict__ rows,
                                        const G* __restrict__ gate, long ld_gate, int size, float eps) {
    dependents_may_start();
    wait_for_earlier_kernels();
    __shared__ float scratch[33];
    const int r = blockIdx.x, g = blockIdx.y;
    const float* part = x + (long)(rows ? rows[r] : r) * ld_x + (long)g * size;
    float sq = 0.0f;
    for (int d = threadIdx.x; d < size; d += blockDim.x) {
        float v = part[d];
        if (GATE == 3) v *= silu_f(to_f32(gate[(long)r * ld_gate + g * size + d]));
        sq = fmaf(v, v, sq);
    }
    const float inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)size + eps);
    for (int d = threadIdx.x; d < size; d += blockDim.x) {
        const int c = g * size + d;
        float v = part[d];
        if (GATE == 3) v *= silu_f(to_f32(gate[(long)r * ld_gate + c]));
        v = v * inv * gain[c];
        if (GATE == 1) v *= sigmoid_f(to_f32(gate[(long)r * ld_gate + c]));
        if (GATE == 2) v *= silu_f(to_f32(gate[(long)r * ld_gate + c]));
        O* o = out + (long)r * ld_out + c;
        if (ADD) *o = from_f32<O>(to_f32(*o) + v);
        else *o = from_f32<O>(v);
    }
}

template <typename O, typename G>
static void launch_grouped_rms_norm(void* out, long ld_out, const float* x, long ld_x, const float* gain, const int* rows,
                                    const void* gate, long ld_gate, int n_rows, int size, int groups, float eps, int add,
                                    int gate_mode, cudaStream_t s) {
    const int threads = size >= 1024 ? 256 : (size >= 256 ? 128 : (size >= 64 ? 64 : 32));
    dim3 grid(n_rows, groups);
    O* o = (O*)out;
    const G* g = (const G*)gate;
    if (add) launch_kernel(g_dependent_launch != 0, grouped_rms_norm_kernel<O, G, true, 0>, dim3(grid), dim3(threads), 0, s, o, ld_out, x, ld_x, gain, rows, g, ld_gate, size, eps);
    else if (gate != nullptr && gate_mode == 3) launch_kernel(g_dependent_launch != 0, grouped_rms_norm_kernel<O, G, false, 3>, dim3(grid), dim3(threads), 0, s, o, ld_out, x, ld_x, gain, rows, g, ld_gate, size, eps);
    else if (gate != nullptr && gate_mode == 2) launch_kernel(g_dependent_launch != 0, grouped_rms_norm_kernel<O, G, false, 2>, dim3(grid), dim3(threads), 0, s, o, ld_out, x, ld_x, gain, rows, g, ld_gate, size, eps);
    else if (gate != nullptr) launch_kernel(g_dependent_launch != 0, grouped_rms_norm_kernel<O, G, false, 1>, dim3(grid), dim3(threads), 0, s, o, ld_out, x, ld_x, gain, rows, g, ld_gate, size, eps);
    else launch_kernel(g_dependent_launch != 0, grouped_rms_norm_kernel<O, G, false, 0>, dim3(grid), dim3(threads), 0, s, o, ld_out, x, ld_x, gain, rows, g, ld_gate, size, eps);
}

// out_dtype / gate_dtype: element types of out and gate.  add != 0: out is fp32 and is added to.
// gate_mode: how the gate enters (1 sigmoid, 2 silu, 3 silu on the input, before the norm).
extern "C" int mllm_sequence_grouped_rms_norm(void* out, long ld_out, const float* x, long ld_x, const float* gain,
                                              const int* rows, const void* gate, long ld_gate, int n_rows, int width,
                                              int groups, float eps, int add, int out_dtype, int gate_dtype, int gate_mode,
                                              void* stream) {
    if (n_rows <= 0) return 0;
    if (groups <= 0 || width <= 0 || width % groups != 0) return fail("grouped_rms_norm: the width is not a multiple of the groups");
    if (groups > 65535) return fail("grouped_rms_norm: too many groups for one launch");
    if (add && (out_dtype != DT_F32 || gate != nullptr)) return fail("grouped_rms_norm: the residual sum is 32-bit and takes no gate");
    if (gate != nullptr && (gate_mode < 1 || gate_mode > 3)) return fail("grouped_rms_norm: unknown gate mode");
    cudaStream_t s = (cudaStream_t)stream;
    const int size = width / groups;
    if (out_dtype == DT_F32 && (gate == nullptr || gate_dtype == DT_F32))
        launch_grouped_rms_norm<float, float>(out, ld_out, x, ld_x, gain, rows, gate, ld_gate, n_rows, size, groups, eps, add, gate_mode, s);
    else if (out_dtype == DT_BF16 && (gate == nullptr || gate_dtype == DT_BF16))
        launch_grouped_rms_norm<bf16, bf16>(out, ld_out, x, ld_x, gain, rows, gate, ld_gate, n_rows, size, groups, eps, add, gate_mode, s);
    else if (out_dtype == DT_F32 && gate_dtype == DT_BF16)
        launch_grouped_rms_norm<float, bf16>(out, ld_out, x, ld_x, gain, rows, gate, ld_gate, n_rows, size, groups, eps, add, gate_mode, s);
    else
        return fail("grouped_rms_norm: unsupported combination of element types");
    return check_launch("grouped_rms_norm_kernel");
}

// ---------------------------------------------------------------------------
// Short causal convolution over time, per channel:
//   out[t, c] = act(identity * h[t, c] + bias[c] + sum_{j < taps} w[c, j] * h[t - (taps - 1) + j, c])
// over the tokens of one request; inputs before this step's portion come from the request's
// state (the last taps - 1 inputs, oldest first, zero before the sequence's start).  `identity`
// (0 or 1) says whether the convolution is added onto its input; `bias` may be null; act is silu
// if `silu` is set.  h and out may have row strides of their own (columns of a wider buffer),
// and out may be h: a block reads its token's earlier rows, so a second buffer is needed only
// when a step brings more than one token of a request (the launcher's caller sees to that).
// One block per token.  A second kernel (one block per entry) then moves the state on; in a step
// of single tokens (writes == 2) the first kernel moves it itself.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void causal_taps_kernel(T* __restrict__ out, long ld_out, const T* __restrict__ h, long ld_h,
                                   const float* __restrict__ w, const float* __restrict__ bias,
                                   float* state, long state_stride, const int* __restrict__ positions,
                                   const int* __restrict__ token_item, const int* __restrict__ item_slot,
                                   const int* __restrict__ item_start, int width, int taps, int identity, int silu,
                                   int moves_state) {
    dependents_may_start();
    wait_for_earlier_kernels();
    const int t = blockIdx.x;
    const int item = token_item[t];
    const int local = positions[t] - item_start[item];          // tokens of this request before t in this step
    float* held = state + (long)item_slot[item] * state_stride;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float mine = to_f32(h[(long)t * ld_h + c]);
        float acc = identity ? mine : 0.0f;
        if (bias != nullptr) acc += bias[c];
        for (int back = taps - 1; back >= 1; back--) {
            float v;
            if (local - back >= 0) v = to_f32(h[(long)(t - back) * ld_h + c]);
            else v = held[(long)(taps - 1 + local - back) * width + c];
            acc = fmaf(w[(long)c * taps + (taps - 1 - back)], v, acc);
        }
        acc = fmaf(w[(long)c * taps + taps - 1], mine, acc);
        if (silu) acc = silu_f(acc);
        out[(long)t * ld_out + c] = from_f32<T>(acc);
        if (moves_state) {
            // a step of single tokens: this thread is the only one that touches the channel's state
            for (int s = 0; s + 1 < taps - 1; s++) held[(long)s * width + c] = held[(long)(s + 1) * width + c];
            if (taps > 1) held[(long)(taps - 2) * width + c] = mine;
        }
    }
}

template <typename T>
__global__ void causal_taps_state_kernel(float* __restrict__ state, long state_stride, const T* __restrict__ h, long ld_h,
                                         const int* __restrict__ item_slot, const int* __restrict__ item_offset,
                                         const int* __restrict__ item_count, int width, int taps) {
    dependents_may_start();
    wait_for_earlier_kernels();
    const int item = blockIdx.x;
    const int count = item_count[item];
    if (count <= 0) return;
    float* held = state + (long)item_slot[item] * state_stride;
    const long first = item_offset[item];
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        // ascending: entry s takes what lay at s + count, which no earlier write has touched
        for (int s = 0; s < taps - 1; s++) {
            const int from = count - (taps - 1) + s;             // index among this step's tokens
            held[(long)s * width + c] = from >= 0 ? to_f32(h[(first + from) * ld_h + c])
                                                  : held[(long)(s + count) * width + c];
        }
    }
}

// A step of single tokens: the norm in groups, the filter and the move of its state as one kernel.
// Every entry brings one token, so all earlier inputs come from the state, and the block that
// reads an entry's state is the only one that writes it.  x: the 32-bit stream; the normed value
// is rounded to the activations' type before it is filtered and kept, as the separate kernels do.
template <typename T>
__global__ void norm_taps_step_kernel(T* __restrict__ out, const float* __restrict__ x, const float* __restrict__ gain,
                                      const float* __restrict__ w, float* __restrict__ state, long state_stride,
                                      const int* __restrict__ token_item, const int* __restrict__ item_slot, int width,
                                      int groups, float eps, int taps, int writes) {
    dependents_may_start();
    wait_for_earlier_kernels();
    extern __shared__ float scale_of_group[];
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    const int size = width / groups;
    const float* row = x + (long)t * width;
    for (int g = warp; g < groups; g += n_warps) {
        float sq = 0.0f;
        for (int d = lane; d < size; d += 32) sq = fmaf(row[g * size + d], row[g * size + d], sq);
        sq = warp_sum(sq);
        if (lane == 0) scale_of_group[g] = 1.0f / sqrtf(sq / (float)size + eps);
    }
    __syncthreads();
    float* held = state + (long)item_slot[token_item[t]] * state_stride;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float mine = to_f32(from_f32<T>(row[c] * scale_of_group[c / size] * gain[c]));
        float acc = mine;
        for (int s = 0; s < taps - 1; s++) acc = fmaf(w[(long)c * taps + s], held[(long)s * width + c], acc);
        acc = fmaf(w[(long)c * taps + taps - 1], mine, acc);
        out[(long)t * width + c] = from_f32<T>(acc);
        if (writes) {
            for (int s = 0; s + 1 < taps - 1; s++) held[(long)s * width + c] = held[(long)(s + 1) * width + c];
            if (taps > 1) held[(long)(taps - 2) * width + c] = mine;
        }
    }
}

extern "C" int mllm_sequence_norm_taps_step(void* out, const float* x, const float* gain, const float* w, float* state,
                                            long state_stride, const int* token_item, const int* item_slot, int n_tokens,
                                            int width, int groups, float eps, int taps, int writes, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (taps < 1 || groups <= 0 || width % groups != 0) return fail("norm_taps_step: bad sizes");
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = width >= 256 ? 256 : 64;
    const size_t shared = (size_t)groups * sizeof(float);
    if (shared > 48 * 1024) return fail("norm_taps_step: too many groups");
    if (dtype == DT_F32)
        launch_kernel(g_dependent_launch != 0, norm_taps_step_kernel<float>, dim3(n_tokens), dim3(threads), shared, s, (float*)out, x,
                      gain, w, state, state_stride, token_item, item_slot, width, groups, eps, taps, writes);
    else if (dtype == DT_BF16)
        launch_kernel(g_dependent_launch != 0, norm_taps_step_kernel<bf16>, dim3(n_tokens), dim3(threads), shared, s, (bf16*)out, x,
                      gain, w, state, state_stride, token_item, item_slot, width, groups, eps, taps, writes);
    else
        return fail("norm_taps_step: unknown dtype");
    return check_launch("norm_taps_step_kernel");
}

// (Not in place: the state's move reads the step's inputs after the filter has run.)
extern "C" int mllm_sequence_causal_taps(void* out, long ld_out, const void* h, long ld_h, const float* w, const float* bias,
                                         float* state, long state_stride, const int* positions, const int* token_item,
                                         const int* item_slot, const int* item_start, const int* item_offset,
                                         const int* item_count, int n_tokens, int n_items, int width, int taps, int writes,
                                         int identity, int silu, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (taps < 1) return fail("causal_taps: at least one tap");
    if (out == h && taps > 1) return fail("causal_taps: the filter does not run in place");
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = width >= 256 ? 256 : 64;
    if (dtype == DT_F32) {
        launch_kernel(g_dependent_launch != 0, causal_taps_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, (float*)out, ld_out,
                      (const float*)h, ld_h, w, bias, state, state_stride, positions, token_item, item_slot, item_start, width,
                      taps, identity, silu, (int)(writes == 2));
        if (writes == 1 && taps > 1)
            launch_kernel(g_dependent_launch != 0, causal_taps_state_kernel<float>, dim3(n_items), dim3(threads), 0, s, state,
                          state_stride, (const float*)h, ld_h, item_slot, item_offset, item_count, width, taps);
    } else if (dtype == DT_BF16) {
        launch_kernel(g_dependent_launch != 0, causal_taps_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, s, (bf16*)out, ld_out,
                      (const bf16*)h, ld_h, w, bias, state, state_stride, positions, token_item, item_slot, item_start, width,
                      taps, identity, silu, (int)(writes == 2));
        if (writes == 1 && taps > 1)
            launch_kernel(g_dependent_launch != 0, causal_taps_state_kernel<bf16>, dim3(n_items), dim3(threads), 0, s, state,
                          state_stride, (const bf16*)h, ld_h, item_slot, item_offset, item_count, width, taps);
    } else {
        return fail("causal_taps: unknown dtype");
    }
    return check_launch("causal_taps_kernel");
}

// ---------------------------------------------------------------------------
// What latent attention keeps of a token, and its queries' rotated parts.
//   down[t] = [rank values | rot values] (fp32): the first are divided by their root mean
//   square and multiplied by `gain` (the latent), the last get rotary positions (the key part
//   all heads share).  Both go into the token's row of the cache pages, [rank + rot] wide.
//   q[t] = per head [dim | rot]: the rot part gets rotary positions and goes, in 32-bit, to
//   q_eff[t, head, rank .. rank + rot) (the first `rank` entries of q_eff are filled by the
//   product with the key expansion).
// Rotary positions: among the first rot_dims entries, pair i turns by position * inv_freq[i] and
// the rest pass unchanged; the pair is (x[2i], x[2i+1]) (layout 0, interleaved) or
// (x[i], x[i + rot_dims/2]) (layout 1, halves).  Angles in 64-bit.
// With `writes` false nothing is stored and `down` is not read (it may be null): an entry that
// reads another entry's rows prepares its queries only.
// One block per token.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void latent_prepare_kernel(T* __restrict__ pages, float* __restrict__ q_eff, const float* __restrict__ down,
                                      const T* __restrict__ q, long ld_q, const float* __restrict__ gain,
                                      const double* __restrict__ inv_freq, const int* __restrict__ positions,
                                      const int* __restrict__ token_item, const int* __restrict__ block_table,
                                      int max_blocks, int page_size, int rank, int rot, int rot_dims, int heads, int dim,
                                      float eps, int writes, int layout) {
    dependents_may_start();
    wait_for_earlier_kernels();
    __shared__ float scratch[33];
    extern __shared__ float turn[];                  // cos[rot_dims / 2], sin[rot_dims / 2]
    const int t = blockIdx.x;
    const int p = positions[t];
    const int half = rot_dims / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        double s, c;
        sincos((double)p * inv_freq[i], &s, &c);
        turn[i] = (float)c;
        turn[half + i] = (float)s;
    }
    // entry e of a rotated part: its pair's index, its partner, and whether it is the pair's second
    auto pair_of = [&](int e, int& i, int& partner) -> bool {
        if (layout == 0) {
            i = e >> 1, partner = e ^ 1;
            return (e & 1) != 0;
        }
        i = e < half ? e : e - half, partner = e < half ? e + half : e - half;
        return e >= half;
    };
    if (writes) {
        const float* mine = down + (long)t * (rank + rot);
        float sq = 0.0f;
        for (int d = threadIdx.x; d < rank; d += blockDim.x) sq = fmaf(mine[d], mine[d], sq);
        const float inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)rank + eps);      // (its barriers also publish turn[])
        const int page = block_table[(long)token_item[t] * max_blocks + p / page_size];
        T* row = pages + ((long)page * page_size + (p % page_size)) * (rank + rot);
        for (int d = threadIdx.x; d < rank; d += blockDim.x) row[d] = from_f32<T>(mine[d] * inv * gain[d]);
        for (int e = threadIdx.x; e < rot; e += blockDim.x) {
            float v = mine[rank + e];
            if (e < 2 * half) {
                int i, partner;
                const bool second = pair_of(e, i, partner);
                const float c = turn[i], s = turn[half + i];
                v = second ? v * c + mine[rank + partner] * s : v * c - mine[rank + partner] * s;
            }
            row[rank + e] = from_f32<T>(v);
        }
    } else {
        __syncthreads();                             // publishes turn[]
    }
    for (int u = threadIdx.x; u < heads * rot; u += blockDim.x) {
        const int head = u / rot, e = u % rot;
        const T* from = q + (long)t * ld_q + (long)head * (dim + rot) + dim;
        float v = to_f32(from[e]);
        if (e < 2 * half) {
            int i, partner;
            const bool second = pair_of(e, i, partner);
            const float c = turn[i], s = turn[half + i];
            v = second ? v * c + to_f32(from[partner]) * s : v * c - to_f32(from[partner]) * s;
        }
        q_eff[((long)t * heads + head) * (rank + rot) + rank + e] = v;
    }
}

extern "C" int mllm_sequence_latent_prepare(void* pages, float* q_eff, const float* down, const void* q, long ld_q,
                                            const float* gain, const double* inv_freq, const int* positions,
                                            const int* token_item, const int* block_table, int max_blocks, int page_size,
                                            int n_tokens, int rank, int rot, int rot_dims, int heads, int dim, float eps,
                                            int writes, int layout, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (layout != 0 && layout != 1) return fail("latent_prepare: the layout of the pairs is 0 (interleaved) or 1 (halves)");
    if (writes && down == nullptr) return fail("latent_prepare: an entry that stores its rows needs its projection");
    if (rot_dims < 0 || rot_dims > rot || rot_dims % 2 != 0) return fail("latent_prepare: rotated dimensions must be even and at most the rotated part");
    cudaStream_t s = (cudaStream_t)stream;
    const size_t shared = (size_t)(rot_dims > 0 ? rot_dims : 1) * sizeof(float);
    if (dtype == DT_F32)
        launch_kernel(g_dependent_launch != 0, latent_prepare_kernel<float>, dim3(n_tokens), dim3(128), shared, s, (float*)pages, q_eff, down, (const float*)q, ld_q, gain, inv_freq,
                                                                   positions, token_item, block_table, max_blocks, page_size,
                                                                   rank, rot, rot_dims, heads, dim, eps, writes, layout);
    else if (dtype == DT_BF16)
        launch_kernel(g_dependent_launch != 0, latent_prepare_kernel<bf16>, dim3(n_tokens), dim3(128), shared, s, (bf16*)pages, q_eff, down, (const bf16*)q, ld_q, gain, inv_freq,
                                                                  positions, token_item, block_table, max_blocks, page_size,
                                                                  rank, rot, rot_dims, heads, dim, eps, writes, layout);
    else
        return fail("latent_prepare: unknown dtype");
    return check_launch("latent_prepare_kernel");
}

// ---------------------------------------------------------------------------
// A batch of products per head: out[t, head, n] = sum_k a[t, head, k] * w[head, n, k].
// a: row stride lda, head stride a_head; out likewise; w [heads, N, K] contiguous.
// The tile scheme of the plain linear kernel (64 x 64, fp32 FMA in order of k).
// ---------------------------------------------------------------------------
template <typename AT, typename WT, typename OT>
__global__ void __launch_bounds__(256)
head_linear_kernel(OT* __restrict__ out, const AT* __restrict__ a, const WT* __restrict__ w, int M, int N, int K, long lda,
                   long ldo, long a_head, long o_head) {
    dependents_may_start();
    wait_for_earlier_kernels();
    constexpr int BM = 64, BN = 64, BK = 16;
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int head = blockIdx.z;
    a += (long)head * a_head;
    out += (long)head * o_head;
    w += (long)head * N * K;
    int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int i = threadIdx.x; i < BM * BK; i += 256) {
            int r = i / BK, c = i % BK;
            int gm = m0 + r, gn = n0 + r, gk = k0 + c;
            As[c][r] = (gm < M && gk < K) ? to_f32(a[(long)gm * lda + gk]) : 0.0f;
            Ws[c][r] = (gn < N && gk < K) ? to_f32(w[(long)gn * K + gk]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            float av[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; i++) av[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) wv[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int gn = n0 + tx * 4 + j;
            if (gn < N) out[(long)gm * ldo + gn] = from_f32<OT>(acc[i][j]);
        }
    }
}

// The same for up to 16 rows (a step of single tokens): a block takes eight output features of one
// head, a warp one of them; the head's rows of `a` lie in shared memory (32-bit), the weight row is
// read once, 16 bytes a lane where K allows it.
template <typename AT, typename WT, typename OT>
__global__ void __launch_bounds__(256)
head_linear_few_rows_kernel(OT* __restrict__ out, const AT* __restrict__ a, const WT* __restrict__ w, int M, int N, int K,
                            long lda, long ldo, long a_head, long o_head) {
    dependents_may_start();
    wait_for_earlier_kernels();
    extern __shared__ float rows[];                 // [M][K]
    const int head = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    a += (long)head * a_head;
    for (int i = threadIdx.x; i < M * K; i += 256) rows[i] = to_f32(a[(long)(i / K) * lda + (i % K)]);
    __syncthreads();
    const int n = blockIdx.x * 8 + warp;
    if (n >= N) return;
    const WT* weights = w + ((long)head * N + n) * K;
    float acc[16];
#pragma unroll
    for (int m = 0; m < 16; m++) acc[m] = 0.0f;
    for (int k = lane; k < K; k += 32) {
        const float x = to_f32(weights[k]);
#pragma unroll
        for (int m = 0; m < 16; m++)
            if (m < M) acc[m] = fmaf(rows[m * K + k], x, acc[m]);
    }
#pragma unroll
    for (int m = 0; m < 16; m++) {
        if (m >= M) break;
        const float total = warp_sum(acc[m]);
        if (lane == 0) out[(long)m * ldo + (long)head * o_head + n] = from_f32<OT>(total);
    }
}

extern "C" int mllm_sequence_head_linear(void* out, const void* a, const void* w, int M, int N, int K, int heads, long lda,
                                         long ldo, long a_head, long o_head, int a_dtype, int w_dtype, int out_dtype,
                                         void* stream) {
    if (M <= 0 || N <= 0 || heads <= 0) return 0;
    if (K <= 0) return fail("head_linear: K must be positive");
    if ((M + 63) / 64 > 65535 || heads > 65535) return fail("head_linear: too many rows or heads for one launch");
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid((N + 63) / 64, (M + 63) / 64, heads);
    const bool few = M <= 16 && (size_t)M * K * sizeof(float) <= 48 * 1024;
    dim3 few_grid((N + 7) / 8, heads);
#define MLLM_HEAD_LINEAR(AT, WT, OT)                                                                                  \
    if (few)                                                                                                          \
        launch_kernel(g_dependent_launch != 0, head_linear_few_rows_kernel<AT, WT, OT>, dim3(few_grid), dim3(256), (size_t)M * K * sizeof(float), s,                  \
            (OT*)out, (const AT*)a, (const WT*)w, M, N, K, lda, ldo, a_head, o_head);                                 \
    else                                                                                                              \
        launch_kernel(g_dependent_launch != 0, head_linear_kernel<AT, WT, OT>, dim3(grid), dim3(256), 0, s, (OT*)out, (const AT*)a, (const WT*)w, M, N, K, lda, ldo,  \
                                                            a_head, o_head)
    if (a_dtype == DT_F32 && w_dtype == DT_F32 && out_dtype == DT_F32) { MLLM_HEAD_LINEAR(float, float, float); }
    else if (a_dtype == DT_BF16 && w_dtype == DT_BF16 && out_dtype == DT_F32) { MLLM_HEAD_LINEAR(bf16, bf16, float); }
    else if (a_dtype == DT_F32 && w_dtype == DT_BF16 && out_dtype == DT_BF16) { MLLM_HEAD_LINEAR(float, bf16, bf16); }
    else if (a_dtype == DT_BF16 && w_dtype == DT_BF16 && out_dtype == DT_BF16) { MLLM_HEAD_LINEAR(bf16, bf16, bf16); }
    else return fail("head_linear: unsupported combination of element types");
#undef MLLM_HEAD_LINEAR
    return check_launch("head_linear_kernel");
}

// ---------------------------------------------------------------------------
// Causal attention over a shared latent, one block per (token, head).
// Every cached token is one row [rank + rot] of the pages; the score of query (t, head)
// against it is q_eff[t, head, :] . row * scale, and the row's first `rank` entries are its
// value.  The query at position p sees positions 0 .. p of its own request, or the last `window`
// of them (window <= 0: all).  Four warps take
// the keys in turn, each with an online softmax (32-bit); their states are merged in a fixed
// order.  out[t, head, :rank] in 32-bit.  R: 32-element pieces of a row a lane may hold.
// ---------------------------------------------------------------------------
template <typename T, int R>
__global__ void __launch_bounds__(128)
latent_attention_kernel(float* __restrict__ out, const float* __restrict__ q_eff, const T* __restrict__ pages,
                        const int* __restrict__ block_table, int max_blocks, const int* __restrict__ positions,
                        const int* __restrict__ token_item, int heads, int rank, int rot, int page_size, float scale,
                        int window) {
    dependents_may_start();
    wait_for_earlier_kernels();
    const int t = blockIdx.x, h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int p = positions[t];
    const int* bt = block_table + (long)token_item[t] * max_blocks;
    const int row_width = rank + rot;
    const float* query = q_eff + ((long)t * heads + h) * row_width;
    float qr[R], acc[R];
#pragma unroll
    for (int i = 0; i < R; i++) {
        const int d = lane + 32 * i;
        qr[i] = d < row_width ? query[d] : 0.0f;
        acc[i] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    for (int j = lo + warp; j <= p; j += 4) {
        const T* row = pages + ((long)bt[j / page_size] * page_size + (j % page_size)) * row_width;
        float kv[R];
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < R; i++) {
            const int d = lane + 32 * i;
            kv[i] = d < row_width ? to_f32(row[d]) : 0.0f;
            s = fmaf(qr[i], kv[i], s);
        }
        s = warp_sum(s) * scale;
        const float m_new = fmaxf(m, s);
        const float c = expf(m - m_new), e = expf(s - m_new);
        l = l * c + e;
#pragma unroll
        for (int i = 0; i < R; i++) acc[i] = acc[i] * c + e * kv[i];       // (entries past `rank` are never stored)
        m = m_new;
    }
    __shared__ float sm_m[4], sm_l[4];
    __shared__ float sm_acc[4][R * 32];
    if (lane == 0) {
        sm_m[warp] = m;
        sm_l[warp] = l;
    }
#pragma unroll
    for (int i = 0; i < R; i++) sm_acc[warp][lane + 32 * i] = acc[i];
    __syncthreads();
    const float big = fmaxf(fmaxf(sm_m[0], sm_m[1]), fmaxf(sm_m[2], sm_m[3]));
    float total = 0.0f, wgt[4];
#pragma unroll
    for (int w = 0; w < 4; w++) {
        wgt[w] = sm_m[w] == -INFINITY ? 0.0f : expf(sm_m[w] - big);
        total += sm_l[w] * wgt[w];
    }
    for (int d = threadIdx.x; d < rank; d += blockDim.x) {
        float o = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; w++) o += sm_acc[w][d] * wgt[w];
        out[((long)t * heads + h) * rank + d] = o / total;
    }
}

template <typename T>
static int launch_latent_attention(float* out, const float* q_eff, const void* pages, const int* block_table, int max_blocks,
                                   const int* positions, const int* token_item, int n_tokens, int heads, int rank, int rot,
                                   int page_size, float scale, int window, cudaStream_t s) {
    dim3 grid(n_tokens, heads);
    const T* pg = (const T*)pages;
    const int pieces = (rank + rot + 31) / 32;
    if (pieces <= 4)
        launch_kernel(g_dependent_launch != 0, latent_attention_kernel<T, 4>, dim3(grid), dim3(128), 0, s, out, q_eff, pg, block_table, max_blocks, positions, token_item, heads, rank, rot, page_size, scale, window);
    else if (pieces <= 8)
        launch_kernel(g_dependent_launch != 0, latent_attention_kernel<T, 8>, dim3(grid), dim3(128), 0, s, out, q_eff, pg, block_table, max_blocks, positions, token_item, heads, rank, rot, page_size, scale, window);
    else if (pieces <= 20)
        launch_kernel(g_dependent_launch != 0, latent_attention_kernel<T, 20>, dim3(grid), dim3(128), 0, s, out, q_eff, pg, block_table, max_blocks, positions, token_item, heads, rank, rot, page_size, scale, window);
    else if (pieces <= 36)
        launch_kernel(g_dependent_launch != 0, latent_attention_kernel<T, 36>, dim3(grid), dim3(128), 0, s, out, q_eff, pg, block_table, max_blocks, positions, token_item, heads, rank, rot, page_size, scale, window);
    else
        return fail("latent_attention: a cached row may hold at most 1152 entries");
    return check_launch("latent_attention_kernel");
}

extern "C" int mllm_sequence_latent_attention(float* out, const float* q_eff, const void* pages, const int* block_table,
                                              int max_blocks, const int* positions, const int* token_item, int n_tokens,
                                              int heads, int rank, int rot, int page_size, float scale, int window,
                                              int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (heads <= 0 || heads > 65535 || rank <= 0 || rot < 0) return fail("latent_attention: bad sizes");
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == DT_F32)
        return launch_latent_attention<float>(out, q_eff, pages, block_table, max_blocks, positions, token_item, n_tokens, heads,
                                              rank, rot, page_size, scale, window, s);
    if (dtype == DT_BF16)
        return launch_latent_attention<bf16>(out, q_eff, pages, block_table, max_blocks, positions, token_item, n_tokens, heads,
                                             rank, rot, page_size, scale, window, s);
    return fail("latent_attention: unknown dtype");
}

// ---------------------------------------------------------------------------
// The same attention in tiles: a block of 256 threads takes 32 query rows that share their
// keys (TQ consecutive tokens of one request x HB heads, TQ * HB = 32) and walks the keys 32
// at a time.  The rows' effective queries (32-bit) and the block of cached rows lie in shared
// memory; scores, softmax and the weighted sum of the latents are 32-bit FMA in register
// tiles (2 x 2 scores per thread; RPT rows x 8 * CT latent columns per thread), so a cached
// row is read once for all heads of HB and all tokens of TQ instead of once per (token, head).
//   prompt portions: `tiles` is the step's work list (records of 8 ints: entry, first row,
//     rows <= 128, position of the first row, part, ...; records with part != 0 are skipped),
//     every record is cut into pieces of TQ tokens (grid.x = records * 128 / TQ);
//   single tokens: tiles is null, TQ = 1, grid.x = tokens, and grid.z = parts: part z takes the
//     z-th run of the token's keys (its context length / parts, rounded up to whole blocks) and
//     leaves (max, sum, unnormalised result) for latent_merge_kernel.
// ---------------------------------------------------------------------------
struct LatentTiledParams {
    void* out;                     // [T, heads * rank], 32-bit or bfloat16
    float* part_out;               // [T, heads, parts, rank]
    float* part_ml;                // [T, heads, parts, 2]
    const float* q_eff;            // [T, heads * (rank + rot)]
    const void* pages;
    const int* block_table; const int* positions; const int* token_item; const int* tiles;
    int max_blocks, page_size, n_tokens, heads, rank, rot, TQ, HB, parts;
    float scale;
    int out_bf16;                  // `out` holds bfloat16 (the expansion that follows then runs on the tensor cores)
    int key_buffers;               // 2: the next block of cached rows is copied (cp.async) while this one is used; 1: no room for that
    int window;                    // a query sees the last `window` positions only (<= 0: all)
};

template <typename T> struct Chunk4;
template <> struct Chunk4<float> { typedef float4 type; };
template <> struct Chunk4<bf16> { typedef uint2 type; };
__device__ __forceinline__ void unpack4(const float4& c, float* v) { v[0] = c.x; v[1] = c.y; v[2] = c.z; v[3] = c.w; }
// An asynchronous copy of BYTES (8 or 16) to shared memory; with `real` false nothing is read and zeros are written.
template <int BYTES>
__device__ __forceinline__ void copy_async(void* to_shared, const void* from_global, bool real) {
    const unsigned to = (unsigned)__cvta_generic_to_shared(to_shared);
    const int bytes = real ? BYTES : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], %2, %3;" ::"r"(to), "l"(from_global), "n"(BYTES), "r"(bytes) : "memory");
}
__device__ __forceinline__ void copies_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int LEFT> __device__ __forceinline__ void copies_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(LEFT) : "memory"); }
__device__ __forceinline__ void unpack4(const uint2& c, float* v) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&c.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&c.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}

template <typename T, int R, int RPT, int CT, int BK>
__global__ void __launch_bounds__(256)
latent_attention_tiled_kernel(LatentTiledParams p) {
    dependents_may_start();
    wait_for_earlier_kernels();
    typedef typename Chunk4<T>::type chunk_t;
    // R rows a block: 32, or 16 for single tokens of models with up to 16 heads (no thread then
    // computes for a row that is nobody's); RW rows per warp in the softmax, RP per thread in the scores
    // BK keys a block: 32, or 64 for prompt portions where they fit (a thread then computes 4 x 2
    // scores from six loads instead of 2 x 2 from four)
    constexpr int CG = 256 / (R / RPT), RW = R / 8, RP = R / 16;
    extern __shared__ __align__(16) unsigned char raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row_width = p.rank + p.rot, ld = row_width + 4;
    float* Qs = reinterpret_cast<float*>(raw);                      // [R][ld]
    float* Ss = Qs + R * ld;                                        // [R][BK + 1]
    float* factor = Ss + R * (BK + 1);                              // [R]: what the sums so far are multiplied by
    float* sums = factor + R;                                       // [R]
    T* Ks = reinterpret_cast<T*>(sums + R);                         // [BK][ld]
    __shared__ int row_position[R];

    int item, first_row, rows, first_position;
    if (p.tiles != nullptr) {
        const int pieces = 128 / p.TQ;
        const int* record = p.tiles + (long)(blockIdx.x / pieces) * 8;
        const int piece = blockIdx.x % pieces;
        if (record[4] != 0 || piece * p.TQ >= record[2]) return;
        item = record[0];
        first_row = record[1] + piece * p.TQ;
        rows = min(p.TQ, record[2] - piece * p.TQ);
        first_position = record[3] + piece * p.TQ;
    } else {
        first_row = blockIdx.x;
        item = p.token_item[first_row];
        rows = 1;
        first_position = p.positions[first_row];
    }
    const int head0 = blockIdx.y * p.HB;
    const int* bt = p.block_table + (long)item * p.max_blocks;
    int key_begin = 0, key_end = first_position + rows;            // keys [key_begin, key_end)
    if (p.window > 0) key_begin = max(0, first_position - p.window + 1);      // (what the block's first row sees first)
    if (p.parts > 1) {
        // the token's own keys, cut into `parts` runs of whole blocks: nothing depends on a length the host knew
        const int per_part = ((key_end - key_begin + p.parts - 1) / p.parts + BK - 1) / BK * BK;
        key_begin += blockIdx.z * per_part;
        key_end = min(key_end, key_begin + per_part);
    }
    const bool empty = key_begin >= key_end;
    // row r of the block: token r / HB of the piece, head head0 + r % HB
    for (int i = tid; i < R * (row_width / 4); i += 256) {
        const int r = i / (row_width / 4), c = (i % (row_width / 4)) * 4;
        const int token = r / p.HB, head = head0 + r % p.HB;
        float4 x = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (token < rows && head < p.heads)
            x = *reinterpret_cast<const float4*>(p.q_eff + ((long)(first_row + token) * p.heads + head) * row_width + c);
        *reinterpret_cast<float4*>(Qs + r * ld + c) = x;
    }
    if (tid < R) {
        const int token = tid / p.HB;
        row_position[tid] = first_position + (token < rows ? token : 0);
    }
    float m_row[RW], l_row[RW];                                     // of rows RW * warp + i, the same in every lane
#pragma unroll
    for (int i = 0; i < RW; i++) {
        m_row[i] = -INFINITY;
        l_row[i] = 0.0f;
    }
    float acc[RPT][8 * CT];
#pragma unroll
    for (int i = 0; i < RPT; i++)
#pragma unroll
        for (int c = 0; c < 8 * CT; c++) acc[i][c] = 0.0f;
    const int rg = tid / CG, cg = tid % CG;
    const int rp = tid >> 4, jp = tid & 15;

    T* const K_first = Ks;
    T* const K_second = Ks + (p.key_buffers == 2 ? BK * ld : 0);
    auto ask = [&](int k0, T* into) {
        for (int i = tid; i < BK * (row_width / 4); i += 256) {
            const int j = i / (row_width / 4), c = (i % (row_width / 4)) * 4;
            const int key = k0 + j;
            const bool real = key < key_end;
            const T* row = reinterpret_cast<const T*>(p.pages);
            if (real) row += ((long)bt[key / p.page_size] * p.page_size + (key % p.page_size)) * row_width + c;
            copy_async<(int)sizeof(chunk_t)>(into + j * ld + c, row, real);
        }
        copies_commit();
    };
    if (p.key_buffers == 2 && !empty) ask(key_begin, K_first);
    int turn = 0;
    for (int k0 = key_begin; k0 < key_end; k0 += BK, turn ^= 1) {
        if (p.key_buffers == 2) {
            Ks = turn ? K_second : K_first;
            // (the block after this one goes where the block before it lay: the barrier that ended the last round freed it)
            if (k0 + BK < key_end) ask(k0 + BK, turn ? K_first : K_second);
            else copies_commit();
            copies_wait<1>();
        } else {
            __syncthreads();                                        // the block before is used up
            ask(k0, Ks);
            copies_wait<0>();
        }
        __syncthreads();                                            // (Qs and row_position are written, too)
        // scores: rows rp, rp + 16 against keys jp, jp + 16
        {
            if constexpr (BK == 64) {
                // rows rq, rq + 8, rq + 16, rq + 24 against keys jq, jq + 32
                const int rq = tid >> 5, jq = tid & 31;
                float sa[4] = {0.0f, 0.0f, 0.0f, 0.0f}, sb[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                for (int d = 0; d < row_width; d += 4) {
                    float ka[4], kb[4];
                    unpack4(*reinterpret_cast<const chunk_t*>(Ks + jq * ld + d), ka);
                    unpack4(*reinterpret_cast<const chunk_t*>(Ks + (jq + 32) * ld + d), kb);
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const float4 q4 = *reinterpret_cast<const float4*>(Qs + (rq + 8 * u) * ld + d);
                        sa[u] = fmaf(q4.x, ka[0], fmaf(q4.y, ka[1], fmaf(q4.z, ka[2], fmaf(q4.w, ka[3], sa[u]))));
                        sb[u] = fmaf(q4.x, kb[0], fmaf(q4.y, kb[1], fmaf(q4.z, kb[2], fmaf(q4.w, kb[3], sb[u]))));
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    Ss[(rq + 8 * u) * (BK + 1) + jq] = sa[u];
                    Ss[(rq + 8 * u) * (BK + 1) + jq + 32] = sb[u];
                }
            } else if constexpr (RP == 2) {
                float s00 = 0.0f, s01 = 0.0f, s10 = 0.0f, s11 = 0.0f;
                for (int d = 0; d < row_width; d += 4) {
                    const float4 qa = *reinterpret_cast<const float4*>(Qs + rp * ld + d);
                    const float4 qb = *reinterpret_cast<const float4*>(Qs + (rp + 16) * ld + d);
                    float ka[4], kb[4];
                    unpack4(*reinterpret_cast<const chunk_t*>(Ks + jp * ld + d), ka);
                    unpack4(*reinterpret_cast<const chunk_t*>(Ks + (jp + 16) * ld + d), kb);
                    s00 = fmaf(qa.x, ka[0], fmaf(qa.y, ka[1], fmaf(qa.z, ka[2], fmaf(qa.w, ka[3], s00))));
                    s01 = fmaf(qa.x, kb[0], fmaf(qa.y, kb[1], fmaf(qa.z, kb[2], fmaf(qa.w, kb[3], s01))));
                    s10 = fmaf(qb.x, ka[0], fmaf(qb.y, ka[1], fmaf(qb.z, ka[2], fmaf(qb.w, ka[3], s10))));
                    s11 = fmaf(qb.x, kb[0], fmaf(qb.y, kb[1], fmaf(qb.z, kb[2], fmaf(qb.w, kb[3], s11))));
                }
                Ss[rp * (BK + 1) + jp] = s00;
                Ss[rp * (BK + 1) + jp + 16] = s01;
                Ss[(rp + 16) * (BK + 1) + jp] = s10;
                Ss[(rp + 16) * (BK + 1) + jp + 16] = s11;
            } else {
                float s0 = 0.0f, s1 = 0.0f;
                for (int d = 0; d < row_width; d += 4) {
                    const float4 qa = *reinterpret_cast<const float4*>(Qs + rp * ld + d);
                    float ka[4], kb[4];
                    unpack4(*reinterpret_cast<const chunk_t*>(Ks + jp * ld + d), ka);
                    unpack4(*reinterpret_cast<const chunk_t*>(Ks + (jp + 16) * ld + d), kb);
                    s0 = fmaf(qa.x, ka[0], fmaf(qa.y, ka[1], fmaf(qa.z, ka[2], fmaf(qa.w, ka[3], s0))));
                    s1 = fmaf(qa.x, kb[0], fmaf(qa.y, kb[1], fmaf(qa.z, kb[2], fmaf(qa.w, kb[3], s1))));
                }
                Ss[rp * (BK + 1) + jp] = s0;
                Ss[rp * (BK + 1) + jp + 16] = s1;
            }
        }
        __syncthreads();
        // softmax, online: warp w owns rows RW w .. RW w + RW - 1, a lane a key
#pragma unroll
        for (int i = 0; i < RW; i++) {
            const int r = warp * RW + i;
            float sc[BK / 32], top = -INFINITY;
#pragma unroll
            for (int u = 0; u < BK / 32; u++) {
                const int key = k0 + lane + 32 * u;
                const bool seen = key < key_end && key <= row_position[r] && (p.window <= 0 || key > row_position[r] - p.window);
                sc[u] = seen ? Ss[r * (BK + 1) + lane + 32 * u] * p.scale : -INFINITY;
                top = fmaxf(top, sc[u]);
            }
            const float m_new = fmaxf(m_row[i], warp_max(top));
            float c = 0.0f, total = 0.0f;
            if (m_new != -INFINITY) c = expf(m_row[i] - m_new);
#pragma unroll
            for (int u = 0; u < BK / 32; u++) {
                const float e = m_new != -INFINITY ? expf(sc[u] - m_new) : 0.0f;
                Ss[r * (BK + 1) + lane + 32 * u] = e;
                total += e;
            }
            l_row[i] = l_row[i] * c + warp_sum(total);
            m_row[i] = m_new;
            if (lane == 0) factor[r] = c;
        }
        __syncthreads();
        // weighted sum of the latents: rows rg * RPT + i, columns (ct * CG + cg) * 8 ..
#pragma unroll
        for (int i = 0; i < RPT; i++) {
            const float c = factor[rg * RPT + i];
#pragma unroll
            for (int x = 0; x < 8 * CT; x++) acc[i][x] *= c;
        }
        for (int j = 0; j < BK; j++) {
            float w[RPT];
#pragma unroll
            for (int i = 0; i < RPT; i++) w[i] = Ss[(rg * RPT + i) * (BK + 1) + j];
#pragma unroll
            for (int ct = 0; ct < CT; ct++) {
                const int c0 = (ct * CG + cg) * 8;
                if (c0 < p.rank) {
                    float v[8];
                    unpack4(*reinterpret_cast<const chunk_t*>(Ks + j * ld + c0), v);
                    unpack4(*reinterpret_cast<const chunk_t*>(Ks + j * ld + c0 + 4), v + 4);
#pragma unroll
                    for (int i = 0; i < RPT; i++)
#pragma unroll
                        for (int x = 0; x < 8; x++) acc[i][ct * 8 + x] = fmaf(w[i], v[x], acc[i][ct * 8 + x]);
                }
            }
        }
        if (p.key_buffers == 2) __syncthreads();                    // this block is used up: the next round may overwrite it
    }
    __syncthreads();
    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < RW; i++) {
            sums[warp * RW + i] = l_row[i];
            factor[warp * RW + i] = m_row[i];
        }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < RPT; i++) {
        const int r = rg * RPT + i;
        const int token = r / p.HB, head = head0 + r % p.HB;
        if (token >= rows || head >= p.heads) continue;
        const long at = (long)(first_row + token) * p.heads + head;
#pragma unroll
        for (int ct = 0; ct < CT; ct++) {
            const int c0 = (ct * CG + cg) * 8;
            if (c0 >= p.rank) continue;
            if (p.parts > 1) {
                float* o = p.part_out + (at * p.parts + blockIdx.z) * p.rank + c0;
#pragma unroll
                for (int x = 0; x < 8; x++) o[x] = empty ? 0.0f : acc[i][ct * 8 + x];
            } else {
                const float inv = 1.0f / sums[r];
                if (p.out_bf16) {
                    bf16* o = reinterpret_cast<bf16*>(p.out) + at * p.rank + c0;
#pragma unroll
                    for (int x = 0; x < 8; x++) o[x] = __float2bfloat16_rn(acc[i][ct * 8 + x] * inv);
                } else {
                    float* o = reinterpret_cast<float*>(p.out) + at * p.rank + c0;
#pragma unroll
                    for (int x = 0; x < 8; x++) o[x] = acc[i][ct * 8 + x] * inv;
                }
            }
        }
        if (p.parts > 1 && cg == 0) {
            p.part_ml[(at * p.parts + blockIdx.z) * 2] = empty ? -INFINITY : factor[r];
            p.part_ml[(at * p.parts + blockIdx.z) * 2 + 1] = empty ? 0.0f : sums[r];
        }
    }
}

// The parts of a (token, head) into one result, in the order of the parts.
__global__ void latent_merge_kernel(void* __restrict__ out, int out_bf16, const float* __restrict__ part_out,
                                    const float* __restrict__ part_ml, int parts, int rank) {
    dependents_may_start();
    wait_for_earlier_kernels();
    __shared__ float weight[32];                 // of each part (there are at most 32), already divided by the sum
    const long at = blockIdx.x;
    if (threadIdx.x < 32) {
        const int z = threadIdx.x;
        const float m = z < parts ? part_ml[(at * parts + z) * 2] : -INFINITY;
        const float l = z < parts ? part_ml[(at * parts + z) * 2 + 1] : 0.0f;
        const float big = warp_max(m);
        const float w = m == -INFINITY ? 0.0f : expf(m - big);
        const float total = warp_sum(l * w);
        weight[z] = w / total;
    }
    __syncthreads();
    const float* mine = part_out + at * parts * rank;
    for (int d = threadIdx.x; d < rank; d += blockDim.x) {
        float o = 0.0f;
#pragma unroll 8
        for (int z = 0; z < parts; z++) o = fmaf(mine[(long)z * rank + d], weight[z], o);
        if (out_bf16) reinterpret_cast<bf16*>(out)[at * rank + d] = __float2bfloat16_rn(o);
        else reinterpret_cast<float*>(out)[at * rank + d] = o;
    }
}

static size_t latent_tiled_shared_bytes(int rows, int row_width, int element_bytes, int key_buffers, int keys = 32) {
    const size_t ld = (size_t)row_width + 4;
    return rows * ld * 4 + rows * (keys + 1) * 4 + 2 * rows * 4 + key_buffers * keys * ld * (size_t)element_bytes;
}

template <typename T, int R, int RPT, int CT, int BK = 32>
static int launch_latent_tiled(const LatentTiledParams& p, dim3 grid, size_t shared, cudaStream_t s) {
    if (shared > 48 * 1024)
        cudaFuncSetAttribute(latent_attention_tiled_kernel<T, R, RPT, CT, BK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    launch_kernel(g_dependent_launch != 0, latent_attention_tiled_kernel<T, R, RPT, CT, BK>, dim3(grid), dim3(256), shared, s, p);
    return check_launch("latent_attention_tiled_kernel");
}

// (a thread's accumulators: RPT rows x 8 CT latent columns; 256 threads cover R rows x the latent)
template <typename T>
static int pick_latent_tiled(const LatentTiledParams& p, int rows, int keys, dim3 grid, size_t shared, cudaStream_t s) {
    if (keys == 64) {
        if (p.rank <= 128) return launch_latent_tiled<T, 32, 2, 1, 64>(p, grid, shared, s);
        if (p.rank <= 256) return launch_latent_tiled<T, 32, 4, 1, 64>(p, grid, shared, s);
        if (p.rank <= 512) return launch_latent_tiled<T, 32, 8, 1, 64>(p, grid, shared, s);
        return launch_latent_tiled<T, 32, 8, 2, 64>(p, grid, shared, s);
    }
    if (rows == 16) {
        if (p.rank <= 128) return launch_latent_tiled<T, 16, 1, 1>(p, grid, shared, s);
        if (p.rank <= 256) return launch_latent_tiled<T, 16, 2, 1>(p, grid, shared, s);
        if (p.rank <= 512) return launch_latent_tiled<T, 16, 4, 1>(p, grid, shared, s);
        return launch_latent_tiled<T, 16, 4, 2>(p, grid, shared, s);
    }
    if (p.rank <= 128) return launch_latent_tiled<T, 32, 2, 1>(p, grid, shared, s);
    if (p.rank <= 256) return launch_latent_tiled<T, 32, 4, 1>(p, grid, shared, s);
    if (p.rank <= 512) return launch_latent_tiled<T, 32, 8, 1>(p, grid, shared, s);
    return launch_latent_tiled<T, 32, 8, 2>(p, grid, shared, s);
}

// n_units: records of `tiles` (prompt portions), or tokens (tiles null: single tokens, in `parts` parts).
extern "C" int mllm_sequence_latent_attention_tiled(const LatentTiledParams* params, int n_units, int dtype, void* stream) {
    LatentTiledParams p = *params;
    if (n_units <= 0) return 0;
    const int row_width = p.rank + p.rot;
    if (row_width % 4 != 0 || p.rank % 8 != 0 || p.rank > 1024) return fail("latent_attention_tiled: the row must be a multiple of 4 and the latent of 8, at most 1024");
    const int rows = p.HB * p.TQ;
    if (p.HB <= 0 || p.TQ <= 0 || (rows != 32 && rows != 16) || 128 % p.TQ != 0) return fail("latent_attention_tiled: a block takes 32 or 16 rows");
    if (p.tiles == nullptr && p.TQ != 1) return fail("latent_attention_tiled: single tokens come one per block");
    if (p.parts < 1 || p.parts > 32 || (p.parts > 1 && (p.tiles != nullptr || p.part_out == nullptr || p.part_ml == nullptr)))
        return fail("latent_attention_tiled: parts are for single tokens and need scratch");
    const int element_bytes = dtype == DT_F32 ? 4 : 2;
    // prompt portions take 64 keys a block where two such blocks, or one, fit beside the queries
    int keys = 32;
    if (p.tiles != nullptr && rows == 32 && latent_tiled_shared_bytes(rows, row_width, element_bytes, 1, 64) <= 220 * 1024) keys = 64;
    p.key_buffers = latent_tiled_shared_bytes(rows, row_width, element_bytes, 2, keys) <= 220 * 1024 ? 2 : 1;
    const size_t shared = latent_tiled_shared_bytes(rows, row_width, element_bytes, p.key_buffers, keys);
    if (shared > 220 * 1024) return fail("latent_attention_tiled: the rows do not fit in shared memory");
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(p.tiles != nullptr ? n_units * (128 / p.TQ) : n_units, (p.heads + p.HB - 1) / p.HB, p.parts);
    int rc;
    if (dtype == DT_F32) rc = pick_latent_tiled<float>(p, rows, keys, grid, shared, s);
    else if (dtype == DT_BF16) rc = pick_latent_tiled<bf16>(p, rows, keys, grid, shared, s);
    else return fail("latent_attention_tiled: unknown dtype");
    if (rc != 0 || p.parts == 1) return rc;
    launch_kernel(g_dependent_launch != 0, latent_merge_kernel, dim3((unsigned)((long)n_units * p.heads)), dim3(128), 0, s, p.out, p.out_bf16, p.part_out, p.part_ml, p.parts, p.rank);
    return check_launch("latent_merge_kernel");
}

// ---------------------------------------------------------------------------
// Matrix memory, token by token.  Per (request, head): S [dim, vdim] with
//   S <- a S + b k v^T,   o = S^T q
// either with a fixed decay per head (a = decay[head], b = 1), or gated and stabilised:
//   li = cap tanh((gi + bias_i) / cap),  lf = logsigmoid(cap tanh((gf + bias_f) / cap)),
//   m' = max(lf + m, li),  a = exp(lf + m - m'),  b = exp(li - m'),
//   n <- a n + b k,   o = S^T q / (max(|n . q|, exp(-m')) + 1e-6)
// with m starting at 0.  q is multiplied by q_scale; with `silu`, q, k and v pass through
// silu first.  State per slot: S [heads, dim, vdim], then (gated) n [heads, dim], m [heads],
// all 32-bit, read at the start of the entry's tokens and written back at their end.
// One block per (entry, head, slice of VS value columns); a thread owns one column of S in
// shared memory and walks the entry's tokens in order; q and k of the next token are fetched
// into the other half of a double buffer meanwhile.  Every slice keeps n and m for itself;
// slice 0 writes them back.
// ---------------------------------------------------------------------------
struct MemoryScanParams {
    float* out; long ld_out;                      // [T, heads * vdim], 32-bit
    const void* q; const void* k; const void* v;  // rows of the activations' element type
    long ld_q, ld_k, ld_v;
    const float* gates; long ld_gates;            // [T, 2 * heads]: input gates, then forget gates (before bias); null: fixed decay
    const float* gate_bias;                       // [2 * heads]
    const float* decay;                           // [heads]
    float* state; long state_stride;
    const int* item_slot; const int* item_offset; const int* item_count;
    int heads, dim, vdim;
    float q_scale, gate_cap;
    int silu, writes;
};

template <typename T, int VS>
__global__ void __launch_bounds__(VS)
memory_scan_kernel(MemoryScanParams p) {
    dependents_may_start();
    wait_for_earlier_kernels();
    extern __shared__ float shared[];
    const int item = blockIdx.x, head = blockIdx.y, v0 = blockIdx.z * VS, tid = threadIdx.x;
    const int count = p.item_count[item];
    if (count <= 0) return;
    const int dim = p.dim, vdim = p.vdim, heads = p.heads;
    const bool gated = p.gates != nullptr;
    const int column = v0 + tid;
    const bool active = column < vdim;
    float* S = shared;                       // [dim][VS]
    float* nvec = S + (long)dim * VS;        // [dim]
    float* qk = nvec + dim;                  // [2][2 * dim]: q then k
    float* held = p.state + (long)p.item_slot[item] * p.state_stride;
    float* S_held = held + (long)head * dim * vdim;
    float* n_held = held + (long)heads * dim * vdim + (long)head * dim;
    float* m_held = held + (long)heads * dim * vdim + (long)heads * dim + head;
    for (int d = 0; d < dim; d++) S[d * VS + tid] = active ? S_held[(long)d * vdim + column] : 0.0f;
    float m = 0.0f;
    if (gated) {
        for (int d = tid; d < dim; d += VS) nvec[d] = n_held[d];
        m = *m_held;
    }
    const long first = p.item_offset[item];
    const T* q = (const T*)p.q + (long)head * dim;
    const T* k = (const T*)p.k + (long)head * dim;
    const T* v = (const T*)p.v + (long)head * vdim;
    auto fetch = [&](long row, float* into) {
        for (int d = tid; d < dim; d += VS) {
            float qd = to_f32(q[row * p.ld_q + d]), kd = to_f32(k[row * p.ld_k + d]);
            if (p.silu) {
                qd = silu_f(qd);
                kd = silu_f(kd);
            }
            into[d] = qd * p.q_scale;
            into[dim + d] = kd;
        }
    };
    fetch(first, qk);
    __syncthreads();
    for (int i = 0; i < count; i++) {
        const long row = first + i;
        const float* qb = qk + (i & 1) * 2 * dim;
        const float* kb = qb + dim;
        float value = active ? to_f32(v[row * p.ld_v + column]) : 0.0f;
        if (p.silu) value = silu_f(value);
        float a, b, m_new = 0.0f;
        if (gated) {
            const float gi = p.gates[row * p.ld_gates + head] + p.gate_bias[head];
            const float gf = p.gates[row * p.ld_gates + heads + head] + p.gate_bias[heads + head];
            const float li = p.gate_cap * tanhf(gi / p.gate_cap);
            const float lf = log_sigmoid_f(p.gate_cap * tanhf(gf / p.gate_cap));
            m_new = fmaxf(lf + m, li);
            a = expf(lf + m - m_new);
            b = expf(li - m_new);
        } else {
            a = p.decay[head];
            b = 1.0f;
        }
        float o = 0.0f, nq = 0.0f, kq = 0.0f;
        const float bv = b * value;
        for (int d = 0; d < dim; d++) {
            const float qd = qb[d], kd = kb[d];
            const float s = fmaf(a, S[d * VS + tid], kd * bv);
            S[d * VS + tid] = s;
            o = fmaf(s, qd, o);
            if (gated) {
                nq = fmaf(nvec[d], qd, nq);
                kq = fmaf(kd, qd, kq);
            }
        }
        if (gated) {
            o /= fmaxf(fabsf(a * nq + b * kq), expf(-m_new)) + 1e-6f;
            m = m_new;
        }
        if (active) p.out[row * p.ld_out + (long)head * vdim + column] = o;
        __syncthreads();                     // every thread is done with nvec and with this token's q and k
        if (gated)
            for (int d = tid; d < dim; d += VS) nvec[d] = fmaf(a, nvec[d], b * kb[d]);
        if (i + 1 < count) fetch(row + 1, qk + ((i + 1) & 1) * 2 * dim);
        __syncthreads();
    }
    if (!p.writes) return;
    if (active)
        for (int d = 0; d < dim; d++) S_held[(long)d * vdim + column] = S[d * VS + tid];
    if (gated && blockIdx.z == 0) {
        for (int d = tid; d < dim; d += VS) n_held[d] = nvec[d];
        if (tid == 0) *m_held = m;
    }
}

extern "C" int mllm_sequence_memory_scan(const MemoryScanParams* params, int n_items, int dtype, void* stream) {
    MemoryScanParams p = *params;
    if (n_items <= 0) return 0;
    if (p.heads <= 0 || p.heads > 65535 || p.dim <= 0 || p.vdim <= 0) return fail("memory_scan: bad sizes");
    constexpr int VS = 32;
    const size_t shared = ((size_t)p.dim * VS + 5 * (size_t)p.dim) * sizeof(float);
    if (shared > 200 * 1024) return fail("memory_scan: the key size is too large for one slice of the state in shared memory");
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(n_items, p.heads, (p.vdim + VS - 1) / VS);
    if (dtype == DT_F32) {
        if (shared > 48 * 1024) cudaFuncSetAttribute(memory_scan_kernel<float, VS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        launch_kernel(g_dependent_launch != 0, memory_scan_kernel<float, VS>, dim3(grid), dim3(VS), shared, s, p);
    } else if (dtype == DT_BF16) {
        if (shared > 48 * 1024) cudaFuncSetAttribute(memory_scan_kernel<bf16, VS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        launch_kernel(g_dependent_launch != 0, memory_scan_kernel<bf16, VS>, dim3(grid), dim3(VS), shared, s, p);
    } else {
        return fail("memory_scan: unknown dtype");
    }
    return check_launch("memory_scan_kernel");
}

// ---------------------------------------------------------------------------
// The same recurrence for prompt portions, a chunk of 32 tokens at a time.  Within a chunk
// nothing is sequential but two prefix scans over the gates: with F_t the sum of the log
// forget gates up to t and b_s = li_s - F_s,
//   M_t = max(m_before, b_0 .. b_t),   m_t = F_t + M_t         (the running maximum)
//   S_t = exp(m_before - M_t) S_before + sum_{s <= t} exp(b_s - M_t) k_s v_s^T
// (every exponent is <= 0), and likewise n_t; with a fixed decay the weights are its powers,
// taken from a table built by repeated multiplication.  So a chunk is three small products in
// 32-bit FMA, spread over 256 threads:  A[t, s] = (q_t . k_s) weight[t, s];
// o_t = carried weight_t (q_t S_before) + sum_s A[t, s] v_s;   S <- weight_last S + sum_s weight[last, s] k_s v_s^T.
// n_t . q_t = carried weight_t (n_before . q_t) + sum_s A[t, s].  One block per (entry, head,
// slice of 32 value columns).  Results differ from the token-by-token kernel by rounding only
// (other order of the sums); decays, gates and state stay 32-bit.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
memory_chunk_kernel(MemoryScanParams p) {
    dependents_may_start();
    wait_for_earlier_kernels();
    constexpr int C = 32, VS = 32;
    extern __shared__ __align__(16) float shared[];
    const int item = blockIdx.x, head = blockIdx.y, v0 = blockIdx.z * VS, tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int count = p.item_count[item];
    if (count <= 0) return;
    const int dim = p.dim, vdim = p.vdim, heads = p.heads;
    const int dimp = (dim + 3) & ~3, ldq = dimp + 4;
    const bool gated = p.gates != nullptr;
    float* qs = shared;                   // [C][ldq]
    float* ks = qs + C * ldq;             // [C][ldq]
    float* vs = ks + C * ldq;             // [C][VS]
    float* S = vs + C * VS;               // [dimp][VS]
    float* A = S + dimp * VS;             // [C][C + 4]
    float* nv = A + C * (C + 4);          // [dimp]
    float* bs = nv + dimp;                // [C]      b_s
    float* Mt = bs + C;                   // [C]      M_t
    float* Fs = Mt + C;                   // [C]      F_t
    float* wt = Fs + C;                   // [C]      weight of the carried state at t
    float* nq = wt + C;                   // [C]      n_before . q_t
    float* dl = nq + C;                   // [C]      weight[last, s]
    float* pw = dl + C;                   // [C + 1]  powers of a fixed decay
    float* held = p.state + (long)p.item_slot[item] * p.state_stride;
    float* S_held = held + (long)head * dim * vdim;
    float* n_held = held + (long)heads * dim * vdim + (long)head * dim;
    float* m_held = held + (long)heads * dim * vdim + (long)heads * dim + head;
    for (int i = tid; i < dimp * VS; i += 256) {
        const int d = i / VS, c = v0 + (i % VS);
        S[i] = (d < dim && c < vdim) ? S_held[(long)d * vdim + c] : 0.0f;
    }
    for (int d = tid; d < dimp; d += 256) nv[d] = (gated && d < dim) ? n_held[d] : 0.0f;
    float m_before = gated ? *m_held : 0.0f;
    if (!gated && tid == 0) {
        float power = 1.0f;
        for (int i = 0; i <= C; i++) {
            pw[i] = power;
            power *= p.decay[head];
        }
    }
    const long first = p.item_offset[item];
    const T* q = (const T*)p.q + (long)head * dim;
    const T* k = (const T*)p.k + (long)head * dim;
    const T* v = (const T*)p.v + (long)head * vdim;
    const int t_mine = tid >> 3, vg = tid & 7;
    // Rows of q, k and v come as 16-byte vectors where the sizes allow it, and the next chunk's are
    // asked for before this chunk is computed, so that their way from memory lies under the sums.
    constexpr int VEC = 16 / (int)sizeof(T), MAXV = 4;
    const int n_vec = dim / VEC;
    const bool vectors = dim % VEC == 0 && vdim % VEC == 0 && p.ld_q % VEC == 0 && p.ld_k % VEC == 0 && p.ld_v % VEC == 0 &&
                         (reinterpret_cast<uintptr_t>(p.q) & 15) == 0 && (reinterpret_cast<uintptr_t>(p.k) & 15) == 0 &&
                         (reinterpret_cast<uintptr_t>(p.v) & 15) == 0 && C * n_vec <= 256 * MAXV;
    uint4 q_next[MAXV], k_next[MAXV], v_next;
    auto ask = [&](int done) {
        const int n = min(C, count - done);
        const long row0 = first + done;
        const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int e = 0; e < MAXV; e++) {
            const int i = tid + e * 256, t = i / n_vec, c = (i % n_vec) * VEC;
            const bool there = i < C * n_vec && t < n;
            q_next[e] = there ? *reinterpret_cast<const uint4*>(q + (row0 + t) * p.ld_q + c) : zero;
            k_next[e] = there ? *reinterpret_cast<const uint4*>(k + (row0 + t) * p.ld_k + c) : zero;
        }
        const int t = tid / (VS / VEC), c = (tid % (VS / VEC)) * VEC;
        v_next = (t < n && v0 + c < vdim) ? *reinterpret_cast<const uint4*>(v + (row0 + t) * p.ld_v + v0 + c) : zero;
    };
    auto unpack = [](const uint4& x, float* out) {
        if (sizeof(T) == 4) {
            out[0] = __uint_as_float(x.x); out[1] = __uint_as_float(x.y); out[2] = __uint_as_float(x.z); out[3] = __uint_as_float(x.w);
        } else {
            const unsigned parts[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float2 two = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&parts[j]));
                out[2 * j] = two.x;
                out[2 * j + 1] = two.y;
            }
        }
    };
    if (vectors) ask(0);
    for (int done = 0; done < count; done += C) {
        const int n = min(C, count - done), last = n - 1;
        const long row0 = first + done;
        __syncthreads();                  // the chunk before is done with everything
        if (vectors) {
#pragma unroll
            for (int e = 0; e < MAXV; e++) {
                const int i = tid + e * 256, t = i / n_vec, c = (i % n_vec) * VEC;
                if (i < C * n_vec) {
                    float qx[VEC], kx[VEC];
                    unpack(q_next[e], qx);
                    unpack(k_next[e], kx);
#pragma unroll
                    for (int x = 0; x < VEC; x++) {
                        qs[t * ldq + c + x] = (p.silu ? silu_f(qx[x]) : qx[x]) * p.q_scale;
                        ks[t * ldq + c + x] = p.silu ? silu_f(kx[x]) : kx[x];
                    }
                }
            }
            if (tid < C * (VS / VEC)) {
                float vx[VEC];
                unpack(v_next, vx);
#pragma unroll
                for (int x = 0; x < VEC; x++) vs[tid * VEC + x] = p.silu ? silu_f(vx[x]) : vx[x];
            }
            if (done + C < count) ask(done + C);
        } else {
        for (int i = tid; i < C * dimp; i += 256) {
            const int t = i / dimp, d = i % dimp;
            float qd = 0.0f, kd = 0.0f;
            if (t < n && d < dim) {
                qd = to_f32(q[(row0 + t) * p.ld_q + d]);
                kd = to_f32(k[(row0 + t) * p.ld_k + d]);
                if (p.silu) {
                    qd = silu_f(qd);
                    kd = silu_f(kd);
                }
                qd *= p.q_scale;
            }
            qs[t * ldq + d] = qd;
            ks[t * ldq + d] = kd;
        }
        for (int i = tid; i < C * VS; i += 256) {
            const int t = i / VS, c = v0 + (i % VS);
            float x = (t < n && c < vdim) ? to_f32(v[(row0 + t) * p.ld_v + c]) : 0.0f;
            if (p.silu) x = silu_f(x);
            vs[i] = x;
        }
        }
        if (gated && warp == 0) {
            float lf = 0.0f, li = -INFINITY;
            if (lane < n) {
                const float gi = p.gates[(row0 + lane) * p.ld_gates + head] + p.gate_bias[head];
                const float gf = p.gates[(row0 + lane) * p.ld_gates + heads + head] + p.gate_bias[heads + head];
                li = p.gate_cap * tanhf(gi / p.gate_cap);
                lf = log_sigmoid_f(p.gate_cap * tanhf(gf / p.gate_cap));
            }
            float F = lf;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float up = __shfl_up_sync(0xffffffffu, F, o);
                if (lane >= o) F += up;
            }
            const float b = li - F;
            float M = b;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float up = __shfl_up_sync(0xffffffffu, M, o);
                if (lane >= o) M = fmaxf(M, up);
            }
            M = fmaxf(M, m_before);
            const float M_last = __shfl_sync(0xffffffffu, M, last);
            bs[lane] = b;
            Mt[lane] = M;
            Fs[lane] = F;
            wt[lane] = expf(m_before - M);
            dl[lane] = lane <= last ? expf(b - M_last) : 0.0f;
        }
        if (!gated && warp == 0) {
            wt[lane] = pw[lane + 1];
            dl[lane] = lane <= last ? pw[last - lane] : 0.0f;
        }
        __syncthreads();
        // A[t, s] = (q_t . k_s) weight[t, s];  nq[t] = n_before . q_t
        {
            const int sg = tid & 7;
            float dot[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            for (int d = 0; d < dimp; d += 4) {
                const float4 q4 = *reinterpret_cast<const float4*>(qs + t_mine * ldq + d);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float4 k4 = *reinterpret_cast<const float4*>(ks + (sg + 8 * i) * ldq + d);
                    dot[i] = fmaf(q4.x, k4.x, fmaf(q4.y, k4.y, fmaf(q4.z, k4.z, fmaf(q4.w, k4.w, dot[i]))));
                }
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int s_at = sg + 8 * i;
                float weight = 0.0f;
                if (s_at <= t_mine && s_at < n) weight = gated ? expf(bs[s_at] - Mt[t_mine]) : pw[t_mine - s_at];
                A[t_mine * (C + 4) + s_at] = dot[i] * weight;
            }
            if (gated) {
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int t = warp * 4 + i;
                    float part = 0.0f;
                    for (int d = lane; d < dimp; d += 32) part = fmaf(nv[d], qs[t * ldq + d], part);
                    part = warp_sum(part);
                    if (lane == 0) nq[t] = part;
                }
            }
        }
        __syncthreads();
        // o_t = carried weight_t (q_t S_before) + sum_s A[t, s] v_s
        {
            float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            for (int d = 0; d < dimp; d += 4) {
                const float4 q4 = *reinterpret_cast<const float4*>(qs + t_mine * ldq + d);
                const float qd[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float4 s4 = *reinterpret_cast<const float4*>(S + (d + i) * VS + vg * 4);
                    acc.x = fmaf(qd[i], s4.x, acc.x);
                    acc.y = fmaf(qd[i], s4.y, acc.y);
                    acc.z = fmaf(qd[i], s4.z, acc.z);
                    acc.w = fmaf(qd[i], s4.w, acc.w);
                }
            }
            const float carried = wt[t_mine];
            acc.x *= carried; acc.y *= carried; acc.z *= carried; acc.w *= carried;
            float row_sum = 0.0f;
            for (int s_at = 0; s_at <= t_mine; s_at++) {
                const float a = A[t_mine * (C + 4) + s_at];
                const float4 v4 = *reinterpret_cast<const float4*>(vs + s_at * VS + vg * 4);
                acc.x = fmaf(a, v4.x, acc.x);
                acc.y = fmaf(a, v4.y, acc.y);
                acc.z = fmaf(a, v4.z, acc.z);
                acc.w = fmaf(a, v4.w, acc.w);
                row_sum += a;
            }
            if (gated) {
                const float below = fmaxf(fabsf(fmaf(carried, nq[t_mine], row_sum)), expf(-(Fs[t_mine] + Mt[t_mine]))) + 1e-6f;
                acc.x /= below; acc.y /= below; acc.z /= below; acc.w /= below;
            }
            if (t_mine < n) {
                float* o = p.out + (row0 + t_mine) * p.ld_out + (long)head * vdim + v0 + vg * 4;
                const int left = vdim - (v0 + vg * 4);
                if (left > 0) o[0] = acc.x;
                if (left > 1) o[1] = acc.y;
                if (left > 2) o[2] = acc.z;
                if (left > 3) o[3] = acc.w;
            }
        }
        __syncthreads();
        // S <- weight_last S + sum_s weight[last, s] k_s v_s^T;  n likewise;  m <- m_last
        {
            const float carried = wt[last];
            for (int d = t_mine; d < dimp; d += 32) {
                float4 s4 = *reinterpret_cast<const float4*>(S + d * VS + vg * 4);
                s4.x *= carried; s4.y *= carried; s4.z *= carried; s4.w *= carried;
                for (int s_at = 0; s_at < n; s_at++) {
                    const float kd = ks[s_at * ldq + d] * dl[s_at];
                    const float4 v4 = *reinterpret_cast<const float4*>(vs + s_at * VS + vg * 4);
                    s4.x = fmaf(kd, v4.x, s4.x);
                    s4.y = fmaf(kd, v4.y, s4.y);
                    s4.z = fmaf(kd, v4.z, s4.z);
                    s4.w = fmaf(kd, v4.w, s4.w);
                }
                *reinterpret_cast<float4*>(S + d * VS + vg * 4) = s4;
            }
            if (gated) {
                for (int d = tid; d < dimp; d += 256) {
                    float x = carried * nv[d];
                    for (int s_at = 0; s_at < n; s_at++) x = fmaf(dl[s_at], ks[s_at * ldq + d], x);
                    nv[d] = x;
                }
                m_before = Fs[last] + Mt[last];
            }
        }
    }
    __syncthreads();
    if (!p.writes) return;
    for (int i = tid; i < dimp * VS; i += 256) {
        const int d = i / VS, c = v0 + (i % VS);
        if (d < dim && c < vdim) S_held[(long)d * vdim + c] = S[i];
    }
    if (gated && blockIdx.z == 0) {
        for (int d = tid; d < dim; d += 256) n_held[d] = nv[d];
        if (tid == 0) *m_held = m_before;
    }
}

static size_t memory_chunk_shared_bytes(int dim) {
    const int dimp = (dim + 3) & ~3, ldq = dimp + 4;
    return ((size_t)2 * 32 * ldq + 32 * 32 + (size_t)dimp * 32 + 32 * 36 + dimp + 6 * 32 + 33) * sizeof(float);
}

// Whether the chunked kernel takes the key size (its chunk of q and k, and a slice of the state, in shared memory).
extern "C" int mllm_sequence_memory_chunk_takes(int dim) { return memory_chunk_shared_bytes(dim) <= 200 * 1024; }

extern "C" int mllm_sequence_memory_chunk(const MemoryScanParams* params, int n_items, int dtype, void* stream) {
    MemoryScanParams p = *params;
    if (n_items <= 0) return 0;
    if (p.heads <= 0 || p.heads > 65535 || p.dim <= 0 || p.vdim <= 0) return fail("memory_chunk: bad sizes");
    const size_t shared = memory_chunk_shared_bytes(p.dim);
    if (shared > 200 * 1024) return fail("memory_chunk: the key size is too large for a chunk in shared memory");
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(n_items, p.heads, (p.vdim + 31) / 32);
    if (dtype == DT_F32) {
        if (shared > 48 * 1024) cudaFuncSetAttribute(memory_chunk_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        launch_kernel(g_dependent_launch != 0, memory_chunk_kernel<float>, dim3(grid), dim3(256), shared, s, p);
    } else if (dtype == DT_BF16) {
        if (shared > 48 * 1024) cudaFuncSetAttribute(memory_chunk_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        launch_kernel(g_dependent_launch != 0, memory_chunk_kernel<bf16>, dim3(grid), dim3(256), shared, s, p);
    } else {
        return fail("memory_chunk: unknown dtype");
    }
    return check_launch("memory_chunk_kernel");
}

// ---------------------------------------------------------------------------
// The chunked recurrence with the chunks side by side.  What ties a chunk to the one before it
// is only the state it starts from, and that follows from the chunks' own sums by a short scan:
//   gates   (gated kind) one warp per (entry, head) walks the entry's gates and leaves, per token:
//           b, M, F, the weight of the carried state, and the token's weight in its chunk's sum
//   sums    per (chunk, head, slice), all at once: D = sum_s weight[last, s] k_s v_s^T  (and of k alone)
//   scan    per (entry, head, slice): S_before(chunk) = S;  S <- carried weight(chunk) S + D(chunk);
//           the chunk's slot in scratch then holds S_before; the entry's state is written at the end
//   read    per (chunk, head, slice), all at once: the scores and outputs of memory_chunk_kernel,
//           from S_before
// Chunks are numbered through the step: entry i owns ceil(count_i / 32) of them; a block finds its
// chunk by walking the entries' counts, so the grid depends on the step's shape only
// (tokens / 32 + entries blocks; those beyond the last chunk leave at once).
// ---------------------------------------------------------------------------
struct MemoryPassParams {
    MemoryScanParams base;
    float* gate_arrays;            // [T, heads, 5]
    float* chunk_state;            // [chunks, heads, dim, vdim]
    float* chunk_norm;             // [chunks, heads, dim]
    int max_chunks, n_items;
};

__device__ __forceinline__ bool find_chunk(const int* __restrict__ item_count, int n_items, int chunk, int& item, int& local) {
    int before = 0;
    for (int i = 0; i < n_items; i++) {
        const int mine = (item_count[i] + 31) >> 5;
        if (chunk < before + mine) {
            item = i;
            local = chunk - before;
            return true;
        }
        before += mine;
    }
    return false;
}

__global__ void __launch_bounds__(32) memory_gates_kernel(MemoryPassParams pp) {
    dependents_may_start();
    wait_for_earlier_kernels();
    const MemoryScanParams& p = pp.base;
    const int item = blockIdx.x, head = blockIdx.y, lane = threadIdx.x, heads = p.heads;
    const int count = p.item_count[item];
    if (count <= 0) return;
    float* m_held = p.state + (long)p.item_slot[item] * p.state_stride + (long)heads * p.dim * p.vdim + (long)heads * p.dim + head;
    float m_before = *m_held;
    const long first = p.item_offset[item];
    for (int done = 0; done < count; done += 32) {
        const int n = min(32, count - done), last = n - 1;
        const long row = first + done + lane;
        float lf = 0.0f, li = -INFINITY;
        if (lane < n) {
            const float gi = p.gates[row * p.ld_gates + head] + p.gate_bias[head];
            const float gf = p.gates[row * p.ld_gates + heads + head] + p.gate_bias[heads + head];
            li = p.gate_cap * tanhf(gi / p.gate_cap);
            lf = log_sigmoid_f(p.gate_cap * tanhf(gf / p.gate_cap));
        }
        float F = lf;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, F, o);
            if (lane >= o) F += up;
        }
        const float b = li - F;
        float M = b;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, M, o);
            if (lane >= o) M = fmaxf(M, up);
        }
        M = fmaxf(M, m_before);
        const float M_last = __shfl_sync(0xffffffffu, M, last), F_last = __shfl_sync(0xffffffffu, F, last);
        if (lane < n) {
            float* mine = pp.gate_arrays + (row * heads + head) * 5;
            mine[0] = b;
            mine[1] = M;
            mine[2] = F;
            mine[3] = expf(m_before - M);
            mine[4] = expf(b - M_last);
        }
        m_before = F_last + M_last;
    }
    if (p.writes && lane == 0) *m_held = m_before;
}

// What a block of the passes over chunks shares: where its chunk lies.
struct ChunkPlace {
    int item, local, n, chunk;
    long row0;
};
__device__ __forceinline__ bool place_chunk(const MemoryPassParams& pp, ChunkPlace& at) {
    at.chunk = blockIdx.x;
    if (!find_chunk(pp.base.item_count, pp.n_items, at.chunk, at.item, at.local)) return false;
    at.n = min(32, pp.base.item_count[at.item] - at.local * 32);
    at.row0 = (long)pp.base.item_offset[at.item] + at.local * 32;
    return true;
}

template <typename T>
__device__ __forceinline__ void load_chunk_rows(const MemoryScanParams& p, const ChunkPlace& at, int head, int v0, float* qs,
                                                float* ks, float* vs, int ldq, int dimp) {
    const T* q = (const T*)p.q + (long)head * p.dim;
    const T* k = (const T*)p.k + (long)head * p.dim;
    const T* v = (const T*)p.v + (long)head * p.vdim;
    for (int i = threadIdx.x; i < 32 * dimp; i += 256) {
        const int t = i / dimp, d = i % dimp;
        float qd = 0.0f, kd = 0.0f;
        if (t < at.n && d < p.dim) {
            if (qs != nullptr) qd = to_f32(q[(at.row0 + t) * p.ld_q + d]);
            kd = to_f32(k[(at.row0 + t) * p.ld_k + d]);
            if (p.silu) {
                qd = silu_f(qd);
                kd = silu_f(kd);
            }
            qd *= p.q_scale;
        }
        if (qs != nullptr) qs[t * ldq + d] = qd;
        ks[t * ldq + d] = kd;
    }
    for (int i = threadIdx.x; i < 32 * 32; i += 256) {
        const int t = i / 32, c = v0 + (i % 32);
        float x = (t < at.n && c < p.vdim) ? to_f32(v[(at.row0 + t) * p.ld_v + c]) : 0.0f;
        if (p.silu) x = silu_f(x);
        vs[i] = x;
    }
}

template <typename T>
__global__ void __launch_bounds__(256) memory_sums_kernel(MemoryPassParams pp) {
    dependents_may_start();
    wait_for_earlier_kernels();
    const MemoryScanParams& p = pp.base;
    ChunkPlace at;
    if (!place_chunk(pp, at)) return;
    extern __shared__ __align__(16) float shared[];
    const int head = blockIdx.y, v0 = blockIdx.z * 32, tid = threadIdx.x, heads = p.heads, dim = p.dim, vdim = p.vdim;
    const int dimp = (dim + 3) & ~3, ldq = dimp + 4, last = at.n - 1;
    const bool gated = p.gates != nullptr;
    float* ks = shared;                    // [32][ldq]
    float* vs = ks + 32 * ldq;             // [32][32]
    float* dl = vs + 32 * 32;              // [32]
    load_chunk_rows<T>(p, at, head, v0, nullptr, ks, vs, ldq, dimp);
    if (tid < 32) {
        float weight = 0.0f;
        if (tid <= last) {
            if (gated) weight = pp.gate_arrays[((at.row0 + tid) * heads + head) * 5 + 4];
            else {
                weight = 1.0f;
                for (int i = 0; i < last - tid; i++) weight *= p.decay[head];
            }
        }
        dl[tid] = weight;
    }
    __syncthreads();
    const int t_mine = tid >> 3, vg = tid & 7;
    float* into = pp.chunk_state + ((long)at.chunk * heads + head) * dim * vdim;
    for (int d = t_mine; d < dim; d += 32) {
        float4 s4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int s_at = 0; s_at < at.n; s_at++) {
            const float kd = ks[s_at * ldq + d] * dl[s_at];
            const float4 v4 = *reinterpret_cast<const float4*>(vs + s_at * 32 + vg * 4);
            s4.x = fmaf(kd, v4.x, s4.x);
            s4.y = fmaf(kd, v4.y, s4.y);
            s4.z = fmaf(kd, v4.z, s4.z);
            s4.w = fmaf(kd, v4.w, s4.w);
        }
        const float out4[4] = {s4.x, s4.y, s4.z, s4.w};
        for (int x = 0; x < 4; x++)
            if (v0 + vg * 4 + x < vdim) into[(long)d * vdim + v0 + vg * 4 + x] = out4[x];
    }
    if (gated && blockIdx.z == 0)
        for (int d = tid; d < dim; d += 256) {
            float x = 0.0f;
            for (int s_at = 0; s_at < at.n; s_at++) x = fmaf(dl[s_at], ks[s_at * ldq + d], x);
            pp.chunk_norm[((long)at.chunk * heads + head) * dim + d] = x;
        }
}

__global__ void __launch_bounds__(256) memory_carry_kernel(MemoryPassParams pp) {
    dependents_may_start();
    wait_for_earlier_kernels();
    const MemoryScanParams& p = pp.base;
    const int item = blockIdx.x, head = blockIdx.y, v0 = blockIdx.z * 32, tid = threadIdx.x;
    const int heads = p.heads, dim = p.dim, vdim = p.vdim;
    const int count = p.item_count[item];
    if (count <= 0) return;
    const bool gated = p.gates != nullptr;
    int chunk = 0;
    for (int i = 0; i < item; i++) chunk += (p.item_count[i] + 31) >> 5;
    const int n_chunks = (count + 31) >> 5;
    float* held = p.state + (long)p.item_slot[item] * p.state_stride;
    float* S_held = held + (long)head * dim * vdim;
    float* n_held = held + (long)heads * dim * vdim + (long)head * dim;
    const long first = p.item_offset[item];
    const int column = v0 + (tid & 31);
    const bool active = column < vdim;
    // a thread owns the entries (d, column) with d = tid / 32 + 8 e.  The chunks' sums do not depend
    // on the state, so they are asked for four chunks ahead: a chunk then costs an addition, not a
    // round trip to L2.
    constexpr int AHEAD = 4;
    auto weight_of = [&](int c) {
        const int n = min(32, count - c * 32);
        if (gated) return pp.gate_arrays[((first + c * 32 + n - 1) * heads + head) * 5 + 3];
        float carried = 1.0f;
        for (int i = 0; i < n; i++) carried *= p.decay[head];
        return carried;
    };
    for (int d0 = tid >> 5; d0 < dim; d0 += 8 * 8) {
        float S[8], ring[AHEAD][8], weights[AHEAD];
        auto ask = [&](int c, int place) {
            const float* slot = pp.chunk_state + ((long)(chunk + c) * heads + head) * dim * vdim;
#pragma unroll
            for (int e = 0; e < 8; e++) {
                const int d = d0 + 8 * e;
                ring[place][e] = (active && d < dim) ? slot[(long)d * vdim + column] : 0.0f;
            }
            weights[place] = weight_of(c);
        };
#pragma unroll
        for (int e = 0; e < 8; e++) {
            const int d = d0 + 8 * e;
            S[e] = (active && d < dim) ? S_held[(long)d * vdim + column] : 0.0f;
        }
#pragma unroll
        for (int a = 0; a < AHEAD; a++)
            if (a < n_chunks) ask(a, a);
        for (int c0 = 0; c0 < n_chunks; c0 += AHEAD) {
#pragma unroll
            for (int a = 0; a < AHEAD; a++) {
                const int c = c0 + a;
                if (c < n_chunks) {
                    float delta[8];
#pragma unroll
                    for (int e = 0; e < 8; e++) delta[e] = ring[a][e];
                    const float carried = weights[a];
                    if (c + AHEAD < n_chunks) ask(c + AHEAD, a);
                    float* slot = pp.chunk_state + ((long)(chunk + c) * heads + head) * dim * vdim;
#pragma unroll
                    for (int e = 0; e < 8; e++) {
                        const int d = d0 + 8 * e;
                        if (active && d < dim) slot[(long)d * vdim + column] = S[e];
                        S[e] = fmaf(carried, S[e], delta[e]);
                    }
                }
            }
        }
        if (p.writes) {
#pragma unroll
            for (int e = 0; e < 8; e++) {
                const int d = d0 + 8 * e;
                if (active && d < dim) S_held[(long)d * vdim + column] = S[e];
            }
        }
    }
    if (gated && blockIdx.z == 0) {
        for (int d = tid; d < dim; d += 256) {
            float x = n_held[d];
            for (int c = 0; c < n_chunks; c++) {
                const int n = min(32, count - c * 32);
                const float carried = pp.gate_arrays[((first + c * 32 + n - 1) * heads + head) * 5 + 3];
                float* slot = pp.chunk_norm + ((long)(chunk + c) * heads + head) * dim + d;
                const float delta = *slot;
                *slot = x;
                x = fmaf(carried, x, delta);
            }
            if (p.writes) n_held[d] = x;
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256) memory_read_kernel(MemoryPassParams pp) {
    dependents_may_start();
    wait_for_earlier_kernels();
    const MemoryScanParams& p = pp.base;
    ChunkPlace at;
    if (!place_chunk(pp, at)) return;
    constexpr int C = 32, VS = 32;
    extern __shared__ __align__(16) float shared[];
    const int head = blockIdx.y, v0 = blockIdx.z * VS, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int heads = p.heads, dim = p.dim, vdim = p.vdim;
    const int dimp = (dim + 3) & ~3, ldq = dimp + 4, n = at.n;
    const bool gated = p.gates != nullptr;
    float* qs = shared;                   // [C][ldq]
    float* ks = qs + C * ldq;             // [C][ldq]
    float* vs = ks + C * ldq;             // [C][VS]
    float* S = vs + C * VS;               // [dimp][VS]
    float* A = S + dimp * VS;             // [C][C + 4]
    float* nv = A + C * (C + 4);          // [dimp]
    float* bs = nv + dimp;                // [C]
    float* Mt = bs + C;                   // [C]
    float* Fs = Mt + C;                   // [C]
    float* wt = Fs + C;                   // [C]
    float* nq = wt + C;                   // [C]
    float* pw = nq + C;                   // [C + 1]
    load_chunk_rows<T>(p, at, head, v0, qs, ks, vs, ldq, dimp);
    const float* before = pp.chunk_state + ((long)at.chunk * heads + head) * dim * vdim;
    for (int i = tid; i < dimp * VS; i += 256) {
        const int d = i / VS, c = v0 + (i % VS);
        S[i] = (d < dim && c < vdim) ? before[(long)d * vdim + c] : 0.0f;
    }
    for (int d = tid; d < dimp; d += 256)
        nv[d] = (gated && d < dim) ? pp.chunk_norm[((long)at.chunk * heads + head) * dim + d] : 0.0f;
    if (warp == 0) {
        if (gated) {
            const float* mine = pp.gate_arrays + ((at.row0 + lane) * heads + head) * 5;
            const bool there = lane < n;
            bs[lane] = there ? mine[0] : -INFINITY;
            Mt[lane] = there ? mine[1] : 0.0f;
            Fs[lane] = there ? mine[2] : 0.0f;
            wt[lane] = there ? mine[3] : 0.0f;
        } else if (lane == 0) {
            float power = 1.0f;
            for (int i = 0; i <= C; i++) {
                pw[i] = power;
                power *= p.decay[head];
            }
        }
    }
    __syncthreads();
    if (!gated && warp == 0) wt[lane] = pw[lane + 1];
    const int t_mine = tid >> 3, vg = tid & 7;
    {
        const int sg = tid & 7;
        float dot[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int d = 0; d < dimp; d += 4) {
            const float4 q4 = *reinterpret_cast<const float4*>(qs + t_mine * ldq + d);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float4 k4 = *reinterpret_cast<const float4*>(ks + (sg + 8 * i) * ldq + d);
                dot[i] = fmaf(q4.x, k4.x, fmaf(q4.y, k4.y, fmaf(q4.z, k4.z, fmaf(q4.w, k4.w, dot[i]))));
            }
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int s_at = sg + 8 * i;
            float weight = 0.0f;
            if (s_at <= t_mine && s_at < n && t_mine < n) weight = gated ? expf(bs[s_at] - Mt[t_mine]) : pw[t_mine - s_at];
            A[t_mine * (C + 4) + s_at] = dot[i] * weight;
        }
        if (gated) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int t = warp * 4 + i;
                float part = 0.0f;
                for (int d = lane; d < dimp; d += 32) part = fmaf(nv[d], qs[t * ldq + d], part);
                part = warp_sum(part);
                if (lane == 0) nq[t] = part;
            }
        }
    }
    __syncthreads();
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int d = 0; d < dimp; d += 4) {
        const float4 q4 = *reinterpret_cast<const float4*>(qs + t_mine * ldq + d);
        const float qd[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float4 s4 = *reinterpret_cast<const float4*>(S + (d + i) * VS + vg * 4);
            acc.x = fmaf(qd[i], s4.x, acc.x);
            acc.y = fmaf(qd[i], s4.y, acc.y);
            acc.z = fmaf(qd[i], s4.z, acc.z);
            acc.w = fmaf(qd[i], s4.w, acc.w);
        }
    }
    const float carried = wt[t_mine];
    acc.x *= carried; acc.y *= carried; acc.z *= carried; acc.w *= carried;
    float row_sum = 0.0f;
    for (int s_at = 0; s_at <= t_mine; s_at++) {
        const float a = A[t_mine * (C + 4) + s_at];
        const float4 v4 = *reinterpret_cast<const float4*>(vs + s_at * VS + vg * 4);
        acc.x = fmaf(a, v4.x, acc.x);
        acc.y = fmaf(a, v4.y, acc.y);
        acc.z = fmaf(a, v4.z, acc.z);
        acc.w = fmaf(a, v4.w, acc.w);
        row_sum += a;
    }
    if (gated) {
        const float below = fmaxf(fabsf(fmaf(carried, nq[t_mine], row_sum)), expf(-(Fs[t_mine] + Mt[t_mine]))) + 1e-6f;
        acc.x /= below; acc.y /= below; acc.z /= below; acc.w /= below;
    }
    if (t_mine < n) {
        float* o = p.out + (at.row0 + t_mine) * p.ld_out + (long)head * vdim + v0 + vg * 4;
        const int left = vdim - (v0 + vg * 4);
        if (left > 0) o[0] = acc.x;
        if (left > 1) o[1] = acc.y;
        if (left > 2) o[2] = acc.z;
        if (left > 3) o[3] = acc.w;
    }
}

// Scratch the passes need, in floats: gate arrays, chunk states, chunk norms.
extern "C" int mllm_sequence_memory_passes(const MemoryPassParams* params, int dtype, void* stream) {
    MemoryPassParams pp = *params;
    const MemoryScanParams& p = pp.base;
    if (pp.n_items <= 0 || pp.max_chunks <= 0) return 0;
    if (p.heads <= 0 || p.heads > 65535 || p.dim <= 0 || p.vdim <= 0) return fail("memory_passes: bad sizes");
    const size_t shared = memory_chunk_shared_bytes(p.dim);
    if (shared > 200 * 1024) return fail("memory_passes: the key size is too large for a chunk in shared memory");
    cudaStream_t s = (cudaStream_t)stream;
    const bool gated = p.gates != nullptr;
    const int slices = (p.vdim + 31) / 32;
    if (gated) launch_kernel(g_dependent_launch != 0, memory_gates_kernel, dim3(dim3(pp.n_items, p.heads)), dim3(32), 0, s, pp);
    dim3 over_chunks(pp.max_chunks, p.heads, slices), over_items(pp.n_items, p.heads, slices);
    if (dtype == DT_F32) {
        if (shared > 48 * 1024) {
            cudaFuncSetAttribute(memory_sums_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
            cudaFuncSetAttribute(memory_read_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        }
        launch_kernel(g_dependent_launch != 0, memory_sums_kernel<float>, dim3(over_chunks), dim3(256), shared, s, pp);
        launch_kernel(g_dependent_launch != 0, memory_carry_kernel, dim3(over_items), dim3(256), 0, s, pp);
        launch_kernel(g_dependent_launch != 0, memory_read_kernel<float>, dim3(over_chunks), dim3(256), shared, s, pp);
    } else if (dtype == DT_BF16) {
        if (shared > 48 * 1024) {
            cudaFuncSetAttribute(memory_sums_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
            cudaFuncSetAttribute(memory_read_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        }
        launch_kernel(g_dependent_launch != 0, memory_sums_kernel<bf16>, dim3(over_chunks), dim3(256), shared, s, pp);
        launch_kernel(g_dependent_launch != 0, memory_carry_kernel, dim3(over_items), dim3(256), 0, s, pp);
        launch_kernel(g_dependent_launch != 0, memory_read_kernel<bf16>, dim3(over_chunks), dim3(256), shared, s, pp);
    } else {
        return fail("memory_passes: unknown dtype");
    }
    return check_launch("memory_passes");
}

// ---------------------------------------------------------------------------
// Weighted sum of all layer results.  kept[t, j, :] holds result j (j < index); the layer's
// own result lies in `hidden`: it is stored as kept[t, index, :], and hidden becomes
// sum_{j <= index} w[j] * kept[t, j, :] (with w null, hidden is only stored: the embedding output).
// ---------------------------------------------------------------------------
__global__ void depth_mix_kernel(float* __restrict__ hidden, float* __restrict__ kept, const float* __restrict__ w, int index,
                                 int planes, int width, long n) {
    dependents_may_start();
    wait_for_earlier_kernels();
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long t = i / width;
    const int c = (int)(i % width);
    float* mine = kept + (t * planes) * width + c;
    const float x = hidden[i];
    mine[(long)index * width] = x;
    if (w == nullptr) return;
    float acc = 0.0f;
    for (int j = 0; j < index; j++) acc = fmaf(w[j], mine[(long)j * width], acc);
    hidden[i] = fmaf(w[index], x, acc);
}

extern "C" int mllm_sequence_depth_mix(float* hidden, float* kept, const float* w, int index, int planes, int n_tokens,
                                       int width, void* stream) {
    if (n_tokens <= 0) return 0;
    if (index < 0 || index >= planes) return fail("depth_mix: the result's index is outside the kept planes");
    const long n = (long)n_tokens * width;
    launch_kernel(g_dependent_launch != 0, depth_mix_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, hidden, kept, w, index, planes, width, n);
    return check_launch("depth_mix_kernel");
}

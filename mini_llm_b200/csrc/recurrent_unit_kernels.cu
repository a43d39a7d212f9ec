// Kernels of layers that norm a sublayer's OUTPUT before the residual sum, of attention with query and
// key norms ahead of rotary positions, and of the real-gated linear recurrent unit:
//   norm_rotary_store  a step's projected queries and keys (32-bit) over their root mean square, times a
//                      gain (over the whole projection, or per head with one gain for all heads), then
//                      rotary positions on the first rot_dims entries of every head (pairs that are
//                      neighbours, or half the rotated entries apart); queries go out in the activations'
//                      type, the keys and the values into their cache pages
//   gated_recurrence   S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t per channel, a_t = exp(-c r_t softplus(lam)),
//                      r_t and i_t the sigmoids of two gates; the output is S_t times gelu(y_t); state and
//                      every gate in 32-bit
//   add_normed_cast    hidden += norm(y) on the 32-bit residual stream, and the new rows rounded to the
//                      activations' type in the same pass (without y: the rounding alone)
//   softcap_rows       x <- cap * tanh(x / cap) on 32-bit rows (logits)
// Every kernel that stores activations is templated on their element type (float: the true 32-bit path;
// bfloat16: the serving path) and is launched as a programmatic dependent of the kernel before it.
#include "common.cuh"

MLLM_DEFINE_ERROR_API(mllm_unit)

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.0f) + log1pf(expf(-fabsf(z))); }

// ---------------------------------------------------------------------------
// Query and key norm, rotary positions, cache store.  A row of `qkv` (32-bit) holds the token's projected
// [q: heads * dim | ... k: kv_heads * dim at k_off | v: kv_heads * vdim at v_off] (v_off may be k_off: the
// values are then the keys as projected, before norm and rotation).  norm_mode 1: q (and k) over the
// root mean square of the whole projection, gains of that size; 2: every head over its own, one gain of
// `dim` entries for all heads; 0: none.  layout 0: entries 2i and 2i+1 turn together; 1: entries i and
// i + rot_dims/2.  Pair i turns by position * inv_freq[i] (the angle in 64-bit, rounded once).  With
// writes == 0 only the queries are made (the keys and values are another layer's).
// One block per token; the token's q and k lie in shared memory in 32-bit.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
norm_rotary_store_kernel(const float* __restrict__ qkv, long ld, int k_off, int v_off, int heads, int kv_heads, int dim,
                         int vdim, T* __restrict__ q_out, long ld_q, const float* __restrict__ q_gain,
                         const float* __restrict__ k_gain, int norm_mode, float eps, int rot_dims, int layout,
                         const double* __restrict__ inv_freq, const int* __restrict__ positions,
                         const int* __restrict__ token_item, const int* __restrict__ block_table, int max_blocks,
                         int page_size, T* __restrict__ k_pages, T* __restrict__ v_pages, int writes) {
    dependents_may_start();
    wait_for_earlier_kernels();
    extern __shared__ float shared[];
    const int all_heads = heads + (writes ? kv_heads : 0);
    const int half = rot_dims / 2;
    float* turn = shared;                       // [rot_dims / 2][2]: cosine, sine
    float* inverse = turn + 2 * half + 2;       // [all_heads]: 1 / root mean square of the head's norm group
    float* scratch = inverse + all_heads;       // [33]
    float* x = scratch + 33;                    // [all_heads * dim]: q heads, then k heads
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    const int p = positions[t];
    const float* row = qkv + (long)t * ld;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        double s, c;
        sincos((double)p * inv_freq[i], &s, &c);
        turn[2 * i] = (float)c;
        turn[2 * i + 1] = (float)s;
    }
    const int q_width = heads * dim, k_width = kv_heads * dim;
    for (int c = threadIdx.x; c < q_width; c += blockDim.x) x[c] = row[c];
    long slot = 0;
    if (writes) {
        slot = (long)block_table[(long)token_item[t] * max_blocks + p / page_size] * page_size + (p % page_size);
        for (int c = threadIdx.x; c < k_width; c += blockDim.x) x[q_width + c] = row[k_off + c];
        // the values leave first: they may be the keys as projected
        for (int c = threadIdx.x; c < kv_heads * vdim; c += blockDim.x)
            v_pages[slot * kv_heads * vdim + c] = from_f32<T>(row[v_off + c]);
    }
    __syncthreads();
    if (norm_mode == 1) {
        float sq = 0.0f, sk = 0.0f;
        for (int c = threadIdx.x; c < q_width; c += blockDim.x) sq = fmaf(x[c], x[c], sq);
        if (writes)
            for (int c = threadIdx.x; c < k_width; c += blockDim.x) sk = fmaf(x[q_width + c], x[q_width + c], sk);
        sq = block_sum(sq, scratch);
        if (writes) sk = block_sum(sk, scratch);
        const float iq = 1.0f / sqrtf(sq / (float)q_width + eps), ik = writes ? 1.0f / sqrtf(sk / (float)k_width + eps) : 0.0f;
        for (int h = threadIdx.x; h < all_heads; h += blockDim.x) inverse[h] = h < heads ? iq : ik;
    } else {
        for (int h = warp; h < all_heads; h += n_warps) {
            float s = 0.0f;
            if (norm_mode == 2)
                for (int d = lane; d < dim; d += 32) s = fmaf(x[h * dim + d], x[h * dim + d], s);
            s = warp_sum(s);
            if (lane == 0) inverse[h] = norm_mode == 2 ? 1.0f / sqrtf(s / (float)dim + eps) : 1.0f;
        }
    }
    __syncthreads();
    // a unit of work: one pair of the rotated part, or one entry of what passes unchanged
    const int units = half + (dim - rot_dims);
    for (int u = threadIdx.x; u < all_heads * units; u += blockDim.x) {
        const int h = u / units, j = u % units;
        const bool is_key = h >= heads;
        const float* gain = is_key ? k_gain : q_gain;
        const int gain_base = norm_mode == 1 ? (is_key ? h - heads : h) * dim : 0;
        const float inv = inverse[h];
        T* dst = is_key ? k_pages + (slot * kv_heads + (h - heads)) * dim : q_out + (long)t * ld_q + (long)h * dim;
        if (j < half) {
            const int ia = layout == 0 ? 2 * j : j, ib = layout == 0 ? 2 * j + 1 : j + half;
            float a = x[h * dim + ia] * inv, b = x[h * dim + ib] * inv;
            if (norm_mode != 0) a *= gain[gain_base + ia], b *= gain[gain_base + ib];
            const float c = turn[2 * j], s = turn[2 * j + 1];
            dst[ia] = from_f32<T>(a * c - b * s);
            dst[ib] = from_f32<T>(b * c + a * s);
        } else {
            const int d = rot_dims + (j - half);
            float a = x[h * dim + d] * inv;
            if (norm_mode != 0) a *= gain[gain_base + d];
            dst[d] = from_f32<T>(a);
        }
    }
}

extern "C" int mllm_unit_norm_rotary_store(const float* qkv, long ld, int k_off, int v_off, int heads, int kv_heads, int dim,
                                           int vdim, void* q_out, long ld_q, const float* q_gain, const float* k_gain,
                                           int norm_mode, float eps, int rot_dims, int layout, const double* inv_freq,
                                           const int* positions, const int* token_item, const int* block_table,
                                           int max_blocks, int page_size, void* k_pages, void* v_pages, int writes,
                                           int n_tokens, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (heads <= 0 || dim <= 0 || (writes && (kv_heads <= 0 || vdim <= 0))) return fail("norm_rotary_store: sizes must be positive");
    if (rot_dims < 0 || rot_dims % 2 != 0 || rot_dims > dim) return fail("norm_rotary_store: an even number of at most dim entries is rotated");
    if (norm_mode < 0 || norm_mode > 2 || layout < 0 || layout > 1) return fail("norm_rotary_store: unknown norm or layout");
    cudaStream_t s = (cudaStream_t)stream;
    const int all_heads = heads + (writes ? kv_heads : 0);
    const size_t shared = sizeof(float) * ((size_t)rot_dims + 2 + all_heads + 33 + (size_t)all_heads * dim);
    if (shared > 200 * 1024) return fail("norm_rotary_store: a token's queries and keys do not fit shared memory");
#define RUN(T)                                                                                                                   \
    do {                                                                                                                         \
        if (shared > 48 * 1024 &&                                                                                                \
            cudaFuncSetAttribute(norm_rotary_store_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared) != cudaSuccess) \
            return fail("norm_rotary_store: the shared memory was refused");                                                     \
        launch_kernel(g_dependent_launch != 0, norm_rotary_store_kernel<T>, dim3(n_tokens), dim3(256), shared, s, qkv, ld, k_off, \
                      v_off, heads, kv_heads, dim, vdim, (T*)q_out, ld_q, q_gain, k_gain, norm_mode, eps, rot_dims, layout,      \
                      inv_freq, positions, token_item, block_table, max_blocks, page_size, (T*)k_pages, (T*)v_pages, writes);    \
    } while (0)
    if (dtype == DT_F32) RUN(float);
    else if (dtype == DT_BF16) RUN(bf16);
    else return fail("norm_rotary_store: unknown dtype");
#undef RUN
    return check_launch("norm_rotary_store_kernel");
}

// ---------------------------------------------------------------------------
// The real-gated linear recurrent unit, per channel c of `inner`:
//   r_t = sigmoid(gates[t, r column of c] + bias_r[c]),  i_t = sigmoid(gates[t, i column of c] + bias_i[c])
//   log a_t = -decay_scale * r_t * softplus(lam[c]),  a_t = exp(log a_t)
//   S_t = a_t S_(t-1) + sqrt(1 - a_t^2) * i_t * u_t,     out_t = S_t * gelu_tanh(y_t)
// with S from the request's slot of `state` (32-bit; zero for a new request, also for its first token).
// `gates` holds, for block b of `block_width` channels, 2 * block_width columns: the r gates of the block's
// channels, then their i gates (the result of one product per block over both gate matrices).
// A block of threads takes UNIT_CHANNELS channels of one entry; its `segments` rows of threads take consecutive runs
// of UNIT_RUN tokens, so the block walks the entry's tokens segments * UNIT_RUN at a time.  Every thread
// computes the gates, a_t and the written value of its run's tokens once (the loads and exponentials of
// different tokens do not wait on one another) and keeps, per token, the product P_t of the run's decays up
// to it and the state s_t the run alone would have built from zero; the runs' (P, s) at their ends are
// chained through shared memory, and then S_t = P_t S_in + s_t.  1 - a^2 is taken as -expm1(2 log a), which
// keeps its digits where a is close to 1.
// ---------------------------------------------------------------------------
constexpr int UNIT_MAX_SEGMENTS = 32;

// (UNIT_RUN tokens a run and UNIT_CHANNELS channels a block: 16 and 16 for steps with prompt portions; 1 and 32 for
// steps of single tokens, where a thread has one token's work and nothing to chain)
template <typename T, int UNIT_RUN, int UNIT_CHANNELS>
__global__ void __launch_bounds__(UNIT_CHANNELS * (UNIT_RUN > 1 ? UNIT_MAX_SEGMENTS : 1))
gated_recurrence_kernel(T* __restrict__ out, long ld_out, const T* __restrict__ u, long ld_u, const T* __restrict__ y, long ld_y,
                        const float* __restrict__ gates, long ld_g, const float* __restrict__ bias_r,
                        const float* __restrict__ bias_i, const float* __restrict__ lam, float decay_scale,
                        float* __restrict__ state, long ld_state, const int* __restrict__ item_slot,
                        const int* __restrict__ item_offset, const int* __restrict__ item_count, int inner, int block_width,
                        int writes) {
    dependents_may_start();
    wait_for_earlier_kernels();
    __shared__ float fold_p[UNIT_MAX_SEGMENTS][UNIT_CHANNELS], fold_s[UNIT_MAX_SEGMENTS][UNIT_CHANNELS];
    __shared__ float carried[UNIT_CHANNELS];
    const int lane_c = threadIdx.x, seg = threadIdx.y, segments = blockDim.y;
    const int c = blockIdx.x * UNIT_CHANNELS + lane_c;
    const int item = blockIdx.y;
    const int count = item_count[item];
    const long first = item_offset[item];
    const bool live = c < inner;
    const int cc = live ? c : 0;                       // (a thread past the last channel computes channel 0 and stores nothing)
    const float rate = -decay_scale * softplus_f(lam[cc]);
    const float br = bias_r[cc], bi = bias_i[cc];
    const long r_col = (long)(cc / block_width) * 2 * block_width + cc % block_width;
    const long i_col = r_col + block_width;
    float* cell = state + (long)item_slot[item] * ld_state + cc;
    if (seg == 0) carried[lane_c] = *cell;
    const int stride = segments * UNIT_RUN;
    for (int base = 0; base < count; base += stride) {
        const int t0 = base + seg * UNIT_RUN;
        float p[UNIT_RUN], s[UNIT_RUN];
        float run_p = 1.0f, run_s = 0.0f;
        // every load of the run is asked for before the first is used (a token past the entry's end reads its last one)
        float gate_r[UNIT_RUN], gate_i[UNIT_RUN], in[UNIT_RUN], side[UNIT_RUN];
#pragma unroll
        for (int k = 0; k < UNIT_RUN; k++) {
            const long row = first + min(t0 + k, count - 1);
            gate_r[k] = gates[row * ld_g + r_col];
            gate_i[k] = gates[row * ld_g + i_col];
            in[k] = to_f32(u[row * ld_u + cc]);
            side[k] = to_f32(y[row * ld_y + cc]);
        }
#pragma unroll
        for (int k = 0; k < UNIT_RUN; k++) {
            const float log_a = rate * sigmoid_f(gate_r[k] + br);
            float a = expf(log_a);
            float b = sqrtf(-expm1f(2.0f * log_a)) * sigmoid_f(gate_i[k] + bi) * in[k];
            if (t0 + k >= count) a = 1.0f, b = 0.0f;
            run_p *= a;
            run_s = fmaf(a, run_s, b);
            p[k] = run_p, s[k] = run_s;
        }
        float s_in;
        if (segments > 1) {
            fold_p[seg][lane_c] = run_p;
            fold_s[seg][lane_c] = run_s;
            __syncthreads();                             // the folds are written; `carried` holds the state before `base`
            s_in = carried[lane_c];
            for (int k = 0; k < seg; k++) s_in = fmaf(fold_p[k][lane_c], s_in, fold_s[k][lane_c]);
        } else {
            s_in = carried[lane_c];
        }
#pragma unroll
        for (int k = 0; k < UNIT_RUN; k++) {
            const int t = t0 + k;
            if (t < count && live)
                out[(first + t) * ld_out + c] = from_f32<T>(fmaf(p[k], s_in, s[k]) * gelu_tanh_f(side[k]));
        }
        if (segments > 1) __syncthreads();               // every thread has read `carried` and the folds
        // the last row of threads ends on the last token of this stretch (an empty run hands its S_in on)
        if (seg == segments - 1) carried[lane_c] = fmaf(run_p, s_in, run_s);
        if (segments > 1 && base + stride < count) __syncthreads();
    }
    if (writes && live && seg == segments - 1) *cell = carried[lane_c];
}

extern "C" int mllm_unit_gated_recurrence(void* out, long ld_out, const void* u, long ld_u, const void* y, long ld_y,
                                          const float* gates, long ld_g, const float* bias_r, const float* bias_i,
                                          const float* lam, float decay_scale, float* state, long ld_state,
                                          const int* item_slot, const int* item_offset, const int* item_count, int inner,
                                          int block_width, int writes, int n_items, int n_tokens, int dtype, void* stream) {
    if (n_items <= 0 || n_tokens <= 0) return 0;
    if (inner <= 0 || block_width <= 0 || inner % block_width != 0) return fail("gated_recurrence: the channels do not split into blocks");
    if (n_items > 65535) return fail("gated_recurrence: too many entries for one launch");
    cudaStream_t s = (cudaStream_t)stream;
    // rows of threads: one for steps of single tokens; else as many runs as the step's mean portion has, up to 32
    const bool single = n_tokens == n_items;
    constexpr int RUN = 16, CHANNELS = 16, SINGLE_CHANNELS = 32;
    int segments = 1;
    const int mean = n_tokens / n_items;
    while (!single && segments < UNIT_MAX_SEGMENTS && segments * RUN < mean) segments *= 2;
    const int channels = single ? SINGLE_CHANNELS : CHANNELS;
    dim3 grid((inner + channels - 1) / channels, n_items), block(channels, segments);
#define RUN_AS(T, R, C)                                                                                                           \
    launch_kernel(g_dependent_launch != 0, gated_recurrence_kernel<T, R, C>, grid, block, 0, s, (T*)out, ld_out, (const T*)u, ld_u, \
                  (const T*)y, ld_y, gates, ld_g, bias_r, bias_i, lam, decay_scale, state, ld_state, item_slot, item_offset,       \
                  item_count, inner, block_width, writes)
    if (dtype == DT_F32) { if (single) RUN_AS(float, 1, SINGLE_CHANNELS); else RUN_AS(float, RUN, CHANNELS); }
    else if (dtype == DT_BF16) { if (single) RUN_AS(bf16, 1, SINGLE_CHANNELS); else RUN_AS(bf16, RUN, CHANNELS); }
    else return fail("gated_recurrence: unknown dtype");
#undef RUN_AS
    return check_launch("gated_recurrence_kernel");
}

// ---------------------------------------------------------------------------
// hidden[t] += y[t] / sqrt(mean(y[t]^2) + eps) * gain, on the 32-bit residual stream (y == nullptr: nothing
// is added); the row as it then is also goes, rounded, to `act` (may be null): what the next sublayer
// reads.  A block per row.
// ---------------------------------------------------------------------------
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
add_normed_cast_kernel(float* __restrict__ hidden, const float* __restrict__ y, const float* __restrict__ gain, float eps,
                       T* __restrict__ act, int width) {
    dependents_may_start();
    wait_for_earlier_kernels();
    __shared__ float scratch[33];
    const long row = blockIdx.x;
    float* h = hidden + row * width;
    const float* v = y != nullptr ? y + row * width : nullptr;
    T* a = act != nullptr ? act + row * width : nullptr;
    if (VEC) {
        // 16-byte vectors; a thread's first vector of y stays in registers between the two passes
        const int n = width / 4;
        float4 kept = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        float inv = 0.0f;
        if (v != nullptr) {
            float sq = 0.0f;
            for (int i = threadIdx.x; i < n; i += blockDim.x) {
                const float4 x = reinterpret_cast<const float4*>(v)[i];
                if (i == (int)threadIdx.x) kept = x;
                sq = fmaf(x.x, x.x, fmaf(x.y, x.y, fmaf(x.z, x.z, fmaf(x.w, x.w, sq))));
            }
            inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)width + eps);
        }
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            float4 sum = reinterpret_cast<const float4*>(h)[i];
            if (v != nullptr) {
                const float4 x = i == (int)threadIdx.x ? kept : reinterpret_cast<const float4*>(v)[i];
                const float4 g = reinterpret_cast<const float4*>(gain)[i];
                sum.x = fmaf(x.x * inv, g.x, sum.x), sum.y = fmaf(x.y * inv, g.y, sum.y);
                sum.z = fmaf(x.z * inv, g.z, sum.z), sum.w = fmaf(x.w * inv, g.w, sum.w);
                reinterpret_cast<float4*>(h)[i] = sum;
            }
            if (a != nullptr) {
                a[4 * i] = from_f32<T>(sum.x), a[4 * i + 1] = from_f32<T>(sum.y);
                a[4 * i + 2] = from_f32<T>(sum.z), a[4 * i + 3] = from_f32<T>(sum.w);
            }
        }
        return;
    }
    float inv = 0.0f;
    if (v != nullptr) {
        float sq = 0.0f;
        for (int c = threadIdx.x; c < width; c += blockDim.x) sq = fmaf(v[c], v[c], sq);
        inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)width + eps);
    }
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float sum = h[c];
        if (v != nullptr) {
            sum = fmaf(v[c] * inv, gain[c], sum);
            h[c] = sum;
        }
        if (a != nullptr) a[c] = from_f32<T>(sum);
    }
}

extern "C" int mllm_unit_add_normed_cast(float* hidden, const float* y, const float* gain, float eps, void* act, int width,
                                         int n_rows, int dtype, void* stream) {
    if (n_rows <= 0) return 0;
    if (width <= 0) return fail("add_normed_cast: the width must be positive");
    if (y != nullptr && gain == nullptr) return fail("add_normed_cast: a norm needs its gain");
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = width % 4 == 0 && (((unsigned long long)hidden | (unsigned long long)y | (unsigned long long)gain) & 15ull) == 0;
    const int threads = width >= 1024 ? 256 : 128;
#define RUN(T, VEC)                                                                                                       \
    launch_kernel(g_dependent_launch != 0, add_normed_cast_kernel<T, VEC>, dim3(n_rows), dim3(threads), 0, s, hidden, y, gain, eps, \
                  (T*)act, width)
    if (dtype == DT_F32) { if (vec) RUN(float, true); else RUN(float, false); }
    else if (dtype == DT_BF16) { if (vec) RUN(bf16, true); else RUN(bf16, false); }
    else return fail("add_normed_cast: unknown dtype");
#undef RUN
    return check_launch("add_normed_cast_kernel");
}

// ---------------------------------------------------------------------------
// x <- cap * tanh(x / cap), 32-bit, in place
// ---------------------------------------------------------------------------
__global__ void softcap_kernel(float* __restrict__ x, float cap, float inv_cap, long n) {
    dependents_may_start();
    wait_for_earlier_kernels();
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] * inv_cap);
}

extern "C" int mllm_unit_softcap(float* x, float cap, long n, void* stream) {
    if (n <= 0) return 0;
    if (!(cap > 0.0f)) return fail("softcap: the cap must be positive");
    long blocks = (n + 255) / 256;
    if (blocks > 4096) blocks = 4096;
    launch_kernel(g_dependent_launch != 0, softcap_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, x, cap, 1.0f / cap, n);
    return check_launch("softcap_kernel");
}

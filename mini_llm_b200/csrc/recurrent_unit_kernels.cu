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
//                      activations' type in the same pass; to_activation: the rounding alone
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
// A block of threads takes 32 channels of one entry; its `segments` rows of threads take consecutive
// runs of the entry's tokens.  With more than one segment every thread first folds its run into
// (A, B), S_out = A S_in + B, the runs' (A, B) are chained through shared memory, and the thread walks
// its run again from its true S_in.  1 - a^2 is taken as -expm1(2 log a), which keeps its digits where a
// is close to 1.
// ---------------------------------------------------------------------------
constexpr int UNIT_CHANNELS = 32;

template <typename T>
__global__ void __launch_bounds__(1024)
gated_recurrence_kernel(T* __restrict__ out, long ld_out, const T* __restrict__ u, long ld_u, const T* __restrict__ y, long ld_y,
                        const float* __restrict__ gates, long ld_g, const float* __restrict__ bias_r,
                        const float* __restrict__ bias_i, const float* __restrict__ lam, float decay_scale,
                        float* __restrict__ state, long ld_state, const int* __restrict__ item_slot,
                        const int* __restrict__ item_offset, const int* __restrict__ item_count, int inner, int block_width,
                        int writes) {
    dependents_may_start();
    wait_for_earlier_kernels();
    __shared__ float fold_a[32][UNIT_CHANNELS], fold_b[32][UNIT_CHANNELS];
    const int c = blockIdx.x * UNIT_CHANNELS + threadIdx.x, seg = threadIdx.y, segments = blockDim.y;
    const int item = blockIdx.y;
    const int count = item_count[item];
    const long first = item_offset[item];
    const bool live = c < inner;
    const int per = (count + segments - 1) / segments;
    const int t0 = min(seg * per, count), t1 = min(t0 + per, count);
    float rate = 0.0f, br = 0.0f, bi = 0.0f;
    long r_col = 0, i_col = 0;
    if (live) {
        rate = -decay_scale * softplus_f(lam[c]);
        br = bias_r[c], bi = bias_i[c];
        r_col = (long)(c / block_width) * 2 * block_width + c % block_width;
        i_col = r_col + block_width;
    }
    float s_in = 0.0f;
    float* cell = state + (long)item_slot[item] * ld_state + c;
    if (segments > 1) {
        float fa = 1.0f, fb = 0.0f;
        if (live)
            for (int t = t0; t < t1; t++) {
                const float* g = gates + (first + t) * ld_g;
                const float log_a = rate * sigmoid_f(g[r_col] + br);
                const float a = expf(log_a);
                const float b = sqrtf(-expm1f(2.0f * log_a)) * sigmoid_f(g[i_col] + bi) * to_f32(u[(first + t) * ld_u + c]);
                fa *= a;
                fb = fmaf(a, fb, b);
            }
        fold_a[seg][threadIdx.x] = fa;
        fold_b[seg][threadIdx.x] = fb;
        __syncthreads();
        if (live) {
            s_in = *cell;
            for (int k = 0; k < seg; k++) s_in = fmaf(fold_a[k][threadIdx.x], s_in, fold_b[k][threadIdx.x]);
        }
    } else if (live) {
        s_in = *cell;
    }
    if (!live) return;
    float s = s_in;
    for (int t = t0; t < t1; t++) {
        const float* g = gates + (first + t) * ld_g;
        const float log_a = rate * sigmoid_f(g[r_col] + br);
        const float a = expf(log_a);
        const float b = sqrtf(-expm1f(2.0f * log_a)) * sigmoid_f(g[i_col] + bi) * to_f32(u[(first + t) * ld_u + c]);
        s = fmaf(a, s, b);
        out[(first + t) * ld_out + c] = from_f32<T>(s * gelu_tanh_f(to_f32(y[(first + t) * ld_y + c])));
    }
    // the last row of threads ends on the entry's last token (an empty run hands its S_in on)
    if (writes && seg == segments - 1) *cell = s;
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
    // rows of threads: one for steps of single tokens; else about 16 tokens a run at the step's mean portion
    int segments = 1;
    const int mean = n_tokens / n_items;
    while (segments < 32 && segments * 16 < mean) segments *= 2;
    dim3 grid((inner + UNIT_CHANNELS - 1) / UNIT_CHANNELS, n_items), block(UNIT_CHANNELS, segments);
    if (dtype == DT_F32)
        launch_kernel(g_dependent_launch != 0, gated_recurrence_kernel<float>, grid, block, 0, s, (float*)out, ld_out, (const float*)u,
                      ld_u, (const float*)y, ld_y, gates, ld_g, bias_r, bias_i, lam, decay_scale, state, ld_state, item_slot,
                      item_offset, item_count, inner, block_width, writes);
    else if (dtype == DT_BF16)
        launch_kernel(g_dependent_launch != 0, gated_recurrence_kernel<bf16>, grid, block, 0, s, (bf16*)out, ld_out, (const bf16*)u,
                      ld_u, (const bf16*)y, ld_y, gates, ld_g, bias_r, bias_i, lam, decay_scale, state, ld_state, item_slot,
                      item_offset, item_count, inner, block_width, writes);
    else
        return fail("gated_recurrence: unknown dtype");
    return check_launch("gated_recurrence_kernel");
}

// ---------------------------------------------------------------------------
// hidden[t] += y[t] / sqrt(mean(y[t]^2) + eps) * gain, on the 32-bit residual stream (y == nullptr: nothing
// is added); the row as it then is also goes, rounded, to `act` (may be null): what the next sublayer
// reads.  A warp per row.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
add_normed_cast_kernel(float* __restrict__ hidden, const float* __restrict__ y, const float* __restrict__ gain, float eps,
                       T* __restrict__ act, int width, int n_rows) {
    dependents_may_start();
    wait_for_earlier_kernels();
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= n_rows) return;
    float* h = hidden + (long)row * width;
    float inv = 0.0f;
    if (y != nullptr) {
        const float* v = y + (long)row * width;
        float sq = 0.0f;
        for (int c = lane; c < width; c += 32) sq = fmaf(v[c], v[c], sq);
        inv = 1.0f / sqrtf(warp_sum(sq) / (float)width + eps);
    }
    for (int c = lane; c < width; c += 32) {
        float sum = h[c];
        if (y != nullptr) {
            sum += y[(long)row * width + c] * inv * gain[c];
            h[c] = sum;
        }
        if (act != nullptr) act[(long)row * width + c] = from_f32<T>(sum);
    }
}

extern "C" int mllm_unit_add_normed_cast(float* hidden, const float* y, const float* gain, float eps, void* act, int width,
                                         int n_rows, int dtype, void* stream) {
    if (n_rows <= 0) return 0;
    if (width <= 0) return fail("add_normed_cast: the width must be positive");
    if (y != nullptr && gain == nullptr) return fail("add_normed_cast: a norm needs its gain");
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid((n_rows + 7) / 8);
    if (dtype == DT_F32)
        launch_kernel(g_dependent_launch != 0, add_normed_cast_kernel<float>, grid, dim3(256), 0, s, hidden, y, gain, eps, (float*)act,
                      width, n_rows);
    else if (dtype == DT_BF16)
        launch_kernel(g_dependent_launch != 0, add_normed_cast_kernel<bf16>, grid, dim3(256), 0, s, hidden, y, gain, eps, (bf16*)act,
                      width, n_rows);
    else
        return fail("add_normed_cast: unknown dtype");
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

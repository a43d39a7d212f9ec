// Kernels of layers that run a softmax attention beside a linear recurrence, and of routed
// feed-forwards:
//   rotary_store      rotary positions (interleaved pairs, a frequency table, an amplitude) on the
//                     step's queries and keys, and the keys and values into their cache pages
//   capped_attention  causal attention over the paged cache with keys and values of different
//                     sizes, a tanh cap on the scores and query heads that share a key/value head;
//                     scores, softmax and the weighted sum of values in 32-bit
//   linear_recurrence S <- a_t S + k_t u_t^T per head with a_t and the write strength b_t per token:
//                     u_t = b_t v_t (state-space form) or u_t = b_t (v_t - (a_t S)^T k_t) (delta rule);
//                     read out after the write; gates, decays and the state in 32-bit
//   route / expert_up / expert_down   a router with sigmoid scores and the largest few experts per
//                     token, gated experts fed the token times its score, a shared expert with an
//                     output gate
//   scaled_add        x += a * u + b * v on the 32-bit residual stream
//   head_norm_store   queries and keys divided by their root mean square per head (no gain), and the
//                     keys and values into their cache pages
// capped_attention also takes a chunked mask (a query sees the keys of its own block of `chunk`
// positions only) and a gate per (token, head) whose sigmoid multiplies the head's result;
// linear_recurrence also takes a decay per key channel instead of one per head.
// Every kernel is templated on the element type of the activations (float: the true 32-bit path;
// bfloat16: the serving path) and is launched as a programmatic dependent of the kernel before it.
#include "common.cuh"

MLLM_DEFINE_ERROR_API(mllm_hybrid)

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.0f) + log1pf(expf(-fabsf(z))); }

// ---------------------------------------------------------------------------
// Rotary positions and the cache store.  A row of `qkv` holds [q: heads * dim | k: kv_heads * dim |
// v: kv_heads * vdim] at the given column offsets.  Among the first rot_dims entries of every
// query and key head, (x[2i], x[2i+1]) turns by position * inv_freq[i]; cosine and sine are
// multiplied by `amplitude`.  Angles are taken in 64-bit, once per token and pair.  Queries and
// keys are rotated in place; keys and values then go to the token's place in the pages.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void rotary_store_kernel(T* __restrict__ qkv, long ld, int k_off, int v_off, int heads, int kv_heads, int dim,
                                    int vdim, int rot_dims, const double* __restrict__ inv_freq, double amplitude,
                                    const int* __restrict__ positions, const int* __restrict__ token_item,
                                    const int* __restrict__ block_table, int max_blocks, int page_size,
                                    T* __restrict__ k_pages, T* __restrict__ v_pages, int writes) {
    dependents_may_start();
    wait_for_earlier_kernels();
    extern __shared__ float turn[];              // [rot_dims / 2][2]: cosine, sine
    const int t = blockIdx.x;
    const int p = positions[t];
    const int half = rot_dims / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        double s, c;
        sincos((double)p * inv_freq[i], &s, &c);
        turn[2 * i] = (float)(c * amplitude);
        turn[2 * i + 1] = (float)(s * amplitude);
    }
    __syncthreads();
    T* row = qkv + (long)t * ld;
    const int page = block_table[(long)token_item[t] * max_blocks + p / page_size];
    const long slot = (long)page * page_size + (p % page_size);
    // queries and keys: pairs of the rotated part, then what passes unchanged
    const int pairs_per_head = dim / 2 + (dim & 1);
    for (int u = threadIdx.x; u < (heads + kv_heads) * pairs_per_head; u += blockDim.x) {
        const int head = u / pairs_per_head, i = u % pairs_per_head;
        const bool is_key = head >= heads;
        T* x = is_key ? row + k_off + (long)(head - heads) * dim : row + (long)head * dim;
        float a = to_f32(x[2 * i]);
        float b = 2 * i + 1 < dim ? to_f32(x[2 * i + 1]) : 0.0f;
        if (i < half) {
            const float c = turn[2 * i], s = turn[2 * i + 1];
            const float ra = a * c - b * s, rb = b * c + a * s;
            a = ra, b = rb;
            x[2 * i] = from_f32<T>(a);
            x[2 * i + 1] = from_f32<T>(b);
        }
        if (is_key && writes) {
            T* dst = k_pages + (slot * kv_heads + (head - heads)) * dim;
            dst[2 * i] = from_f32<T>(a);
            if (2 * i + 1 < dim) dst[2 * i + 1] = from_f32<T>(b);
        }
    }
    if (writes)
        for (int c = threadIdx.x; c < kv_heads * vdim; c += blockDim.x)
            v_pages[slot * kv_heads * vdim + c] = row[v_off + c];
}

extern "C" int mllm_hybrid_rotary_store(void* qkv, long ld, int k_off, int v_off, int heads, int kv_heads, int dim, int vdim,
                                        int rot_dims, const double* inv_freq, double amplitude, const int* positions,
                                        const int* token_item, const int* block_table, int max_blocks, int page_size,
                                        void* k_pages, void* v_pages, int writes, int n_tokens, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (rot_dims < 0 || rot_dims % 2 != 0 || rot_dims > dim) return fail("rotary_store: an even number of at most dim entries is rotated");
    cudaStream_t s = (cudaStream_t)stream;
    const size_t shared = (size_t)(rot_dims + 2) * sizeof(float);
    if (dtype == DT_F32)
        launch_kernel(g_dependent_launch != 0, rotary_store_kernel<float>, dim3(n_tokens), dim3(128), shared, s, (float*)qkv, ld,
                      k_off, v_off, heads, kv_heads, dim, vdim, rot_dims, inv_freq, amplitude, positions, token_item, block_table,
                      max_blocks, page_size, (float*)k_pages, (float*)v_pages, writes);
    else if (dtype == DT_BF16)
        launch_kernel(g_dependent_launch != 0, rotary_store_kernel<bf16>, dim3(n_tokens), dim3(128), shared, s, (bf16*)qkv, ld,
                      k_off, v_off, heads, kv_heads, dim, vdim, rot_dims, inv_freq, amplitude, positions, token_item, block_table,
                      max_blocks, page_size, (bf16*)k_pages, (bf16*)v_pages, writes);
    else
        return fail("rotary_store: unknown dtype");
    return check_launch("rotary_store_kernel");
}

// ---------------------------------------------------------------------------
// Queries and keys over their root mean square, per head and without a gain:
// x / sqrt(mean(x^2) + eps) over the head's `dim` entries, in place; the normed keys and the values
// then go to the token's place in the pages.  A row of `qkv` is laid out as for rotary_store.  One
// block per token, a warp per head in turn; sums in 32-bit.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
head_norm_store_kernel(T* __restrict__ qkv, long ld, int k_off, int v_off, int heads, int kv_heads, int dim, int vdim,
                       float eps, const int* __restrict__ positions, const int* __restrict__ token_item,
                       const int* __restrict__ block_table, int max_blocks, int page_size, T* __restrict__ k_pages,
                       T* __restrict__ v_pages, int writes) {
    dependents_may_start();
    wait_for_earlier_kernels();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int p = positions[t];
    T* row = qkv + (long)t * ld;
    long slot = 0;
    if (writes) slot = (long)block_table[(long)token_item[t] * max_blocks + p / page_size] * page_size + (p % page_size);
    for (int head = warp; head < heads + kv_heads; head += 4) {
        const bool is_key = head >= heads;
        T* x = is_key ? row + k_off + (long)(head - heads) * dim : row + (long)head * dim;
        float sq = 0.0f;
        for (int d = lane; d < dim; d += 32) {
            const float v = to_f32(x[d]);
            sq = fmaf(v, v, sq);
        }
        const float inv = eps >= 0.0f ? 1.0f / sqrtf(warp_sum(sq) / (float)dim + eps) : 1.0f;      // (eps < 0: stored as they are)
        T* dst = k_pages + (slot * kv_heads + (head - heads)) * dim;
        for (int d = lane; d < dim; d += 32) {
            const T v = from_f32<T>(to_f32(x[d]) * inv);
            x[d] = v;
            if (is_key && writes) dst[d] = v;
        }
    }
    if (writes)
        for (int c = threadIdx.x; c < kv_heads * vdim; c += blockDim.x) v_pages[slot * kv_heads * vdim + c] = row[v_off + c];
}

extern "C" int mllm_hybrid_head_norm_store(void* qkv, long ld, int k_off, int v_off, int heads, int kv_heads, int dim, int vdim,
                                           float eps, const int* positions, const int* token_item, const int* block_table,
                                           int max_blocks, int page_size, void* k_pages, void* v_pages, int writes, int n_tokens,
                                           int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (heads <= 0 || kv_heads <= 0 || dim <= 0 || vdim <= 0) return fail("head_norm_store: sizes must be positive");
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == DT_F32)
        launch_kernel(g_dependent_launch != 0, head_norm_store_kernel<float>, dim3(n_tokens), dim3(128), 0, s, (float*)qkv, ld, k_off,
                      v_off, heads, kv_heads, dim, vdim, eps, positions, token_item, block_table, max_blocks, page_size,
                      (float*)k_pages, (float*)v_pages, writes);
    else if (dtype == DT_BF16)
        launch_kernel(g_dependent_launch != 0, head_norm_store_kernel<bf16>, dim3(n_tokens), dim3(128), 0, s, (bf16*)qkv, ld, k_off,
                      v_off, heads, kv_heads, dim, vdim, eps, positions, token_item, block_table, max_blocks, page_size,
                      (bf16*)k_pages, (bf16*)v_pages, writes);
    else
        return fail("head_norm_store: unknown dtype");
    return check_launch("head_norm_store_kernel");
}

// ---------------------------------------------------------------------------
// Causal attention with capped scores, one block per (token, head): the plain form, which takes
// every size.  score = cap * tanh((q . k) * scale / cap) (cap <= 0: no cap); the query at position
// p sees keys max(0, p - window + 1) .. p (window <= 0: all).  Four warps take the keys in turn,
// each with an online softmax; their states are merged in a fixed order.
// ---------------------------------------------------------------------------
constexpr int CAP_MAX_HEAD = 256;

__device__ __forceinline__ float capped(float s, float cap, float inv_cap) { return cap > 0.0f ? cap * tanhf(s * inv_cap) : s; }

// The first key the query at position p sees: the last `window` positions (window <= 0: all), and
// within its own block of `chunk` positions counted from 0 (chunk <= 0: no blocks).
__device__ __forceinline__ int first_visible(int p, int window, int chunk) {
    int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    if (chunk > 0) lo = max(lo, (p / chunk) * chunk);
    return lo;
}

template <typename T>
__global__ void __launch_bounds__(128)
capped_attention_plain_kernel(T* __restrict__ out, long ld_out, const T* __restrict__ q, long ld_q,
                              const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                              const int* __restrict__ block_table, int max_blocks, const int* __restrict__ positions,
                              const int* __restrict__ token_item, int n_heads, int n_kv_heads, int dim, int vdim,
                              int page_size, float scale, float cap, int window, int chunk,
                              const float* __restrict__ gate, long ld_gate, const float* __restrict__ sink) {
    dependents_may_start();
    wait_for_earlier_kernels();
    constexpr int R = CAP_MAX_HEAD / 32;
    const int t = blockIdx.x, h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int p = positions[t];
    const int* bt = block_table + (long)token_item[t] * max_blocks;
    const int hk = h / (n_heads / n_kv_heads);
    const float inv_cap = cap > 0.0f ? 1.0f / cap : 0.0f;
    float qr[R], acc[R];
#pragma unroll
    for (int i = 0; i < R; i++) {
        const int d = lane + 32 * i;
        qr[i] = d < dim ? to_f32(q[(long)t * ld_q + (long)h * dim + d]) : 0.0f;
        acc[i] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    const int lo = first_visible(p, window, chunk);
    for (int j = lo + warp; j <= p; j += 4) {
        const long slot = (long)bt[j / page_size] * page_size + (j % page_size);
        const T* kr = k_pages + (slot * n_kv_heads + hk) * dim;
        const T* vr = v_pages + (slot * n_kv_heads + hk) * vdim;
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < R; i++) {
            const int d = lane + 32 * i;
            if (d < dim) s = fmaf(qr[i], to_f32(kr[d]), s);
        }
        s = capped(warp_sum(s) * scale, cap, inv_cap);
        const float m_new = fmaxf(m, s);
        const float c = expf(m - m_new), e = expf(s - m_new);
        l = l * c + e;
#pragma unroll
        for (int i = 0; i < R; i++) {
            const int d = lane + 32 * i;
            if (d < vdim) acc[i] = acc[i] * c + e * to_f32(vr[d]);
        }
        m = m_new;
    }
    __shared__ float sm_m[4], sm_l[4];
    __shared__ float sm_acc[4][CAP_MAX_HEAD];
    if (lane == 0) sm_m[warp] = m, sm_l[warp] = l;
#pragma unroll
    for (int i = 0; i < R; i++) {
        const int d = lane + 32 * i;
        if (d < vdim) sm_acc[warp][d] = acc[i];
    }
    __syncthreads();
    float big = fmaxf(fmaxf(sm_m[0], sm_m[1]), fmaxf(sm_m[2], sm_m[3]));
    // a sink: one more term exp(sink[h]) in the denominator, with no key and no value
    if (sink != nullptr) big = fmaxf(big, sink[h]);
    float total = sink != nullptr ? expf(sink[h] - big) : 0.0f, wgt[4];
#pragma unroll
    for (int w = 0; w < 4; w++) {
        wgt[w] = sm_m[w] == -INFINITY ? 0.0f : expf(sm_m[w] - big);
        total += sm_l[w] * wgt[w];
    }
    const float open = gate != nullptr ? sigmoid_f(gate[(long)t * ld_gate + h]) : 1.0f;
    for (int d = threadIdx.x; d < vdim; d += blockDim.x) {
        float o = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; w++) o += sm_acc[w][d] * wgt[w];
        out[(long)t * ld_out + (long)h * vdim + d] = from_f32<T>(o / total * open);
    }
}

// ---------------------------------------------------------------------------
// The same attention in tiles, for steps with prompt portions.  A block takes consecutive tokens
// of the step and up to HC query heads of one key/value head: 8 * R (token, head) rows, R a warp
// (R = 2 or 4: a step with many rows lets more of them share a block's keys).  Tokens of
// one request that lie side by side share every block of 32 cached keys and values, which the
// block brings into shared memory once, in 32-bit, as 16-byte vectors asked for a block ahead.
// Within a warp the lanes take the 32 keys of a block for the scores (a key's entries are read
// once for all R rows) and the value entries for the weighted sum (a value's entry is read once
// for all R rows); scores, maxima, sums and weights are 32-bit.  A tile whose tokens belong to
// several requests takes the requests one after the other.
// ---------------------------------------------------------------------------
constexpr int TILE_KEYS = 32;
constexpr int TILE_WARPS = 8;

// sixteen bytes of activations as 32-bit floats into shared memory
template <typename T> __device__ __forceinline__ void widen(const uint4& v, float* dst);
template <> __device__ __forceinline__ void widen<float>(const uint4& v, float* dst) {
    *reinterpret_cast<float4*>(dst) = make_float4(__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z), __uint_as_float(v.w));
}
template <> __device__ __forceinline__ void widen<bf16>(const uint4& v, float* dst) {
    // a bfloat16 is the upper half of the float it stands for
    *reinterpret_cast<float4*>(dst) = make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u),
                                                  __uint_as_float(v.y << 16), __uint_as_float(v.y & 0xffff0000u));
    *reinterpret_cast<float4*>(dst + 4) = make_float4(__uint_as_float(v.z << 16), __uint_as_float(v.z & 0xffff0000u),
                                                      __uint_as_float(v.w << 16), __uint_as_float(v.w & 0xffff0000u));
}

template <typename T, int R, int SIZE>      // rows a warp; the least of 64, 128, 256 that holds the key and the value size
__global__ void __launch_bounds__(TILE_WARPS * 32, R <= 4 && SIZE <= 128 ? 2 : 1)
capped_attention_tiled_kernel(T* __restrict__ out, long ld_out, const T* __restrict__ q, long ld_q,
                              const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                              const int* __restrict__ block_table, int max_blocks, const int* __restrict__ positions,
                              const int* __restrict__ token_item, int n_tokens, int n_heads, int n_kv_heads, int dim,
                              int vdim, int page_size, float scale, float cap, int window, int chunk,
                              const float* __restrict__ gate, long ld_gate, const float* __restrict__ sink,
                              int tokens_per_block, int heads_per_block) {
    dependents_may_start();
    wait_for_earlier_kernels();
    constexpr int ROWS = TILE_WARPS * R;
    constexpr int VPL = SIZE / 32;                           // value entries a lane
    extern __shared__ float shared[];
    const int kd = dim + 4;                                  // padded key row: lanes read rows, four entries at a time
    float* q_rows = shared;                                  // [ROWS][dim]
    float* keys = q_rows + ROWS * dim;                       // [TILE_KEYS][kd]
    float* values = keys + TILE_KEYS * kd;                   // [TILE_KEYS][vdim]
    float* weights = values + TILE_KEYS * vdim;              // [TILE_WARPS][TILE_KEYS][R]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = n_heads / n_kv_heads;
    const int chunks = (group + heads_per_block - 1) / heads_per_block;
    const int hk = blockIdx.y / chunks;
    const int first_head = hk * group + (blockIdx.y % chunks) * heads_per_block;
    const int n_heads_here = min(heads_per_block, hk * group + group - first_head);
    const int first_token = blockIdx.x * tokens_per_block;
    const int n_tok = min(tokens_per_block, n_tokens - first_token);
    const int n_rows = n_tok * n_heads_here;
    const float inv_cap = cap > 0.0f ? 1.0f / cap : 0.0f;

    // this warp's rows: r = warp + s * TILE_WARPS; row r = (token r / heads, head r % heads)
    int row_pos[R], row_item[R];
    float m[R], l[R], acc[R][VPL];
#pragma unroll
    for (int s = 0; s < R; s++) {
        const int r = warp + s * TILE_WARPS;
        const bool live = r < n_rows;
        const int token = live ? first_token + r / n_heads_here : 0;
        row_pos[s] = live ? positions[token] : -1;
        row_item[s] = live ? token_item[token] : -1;
        m[s] = -INFINITY, l[s] = 0.0f;
#pragma unroll
        for (int i = 0; i < VPL; i++) acc[s][i] = 0.0f;
    }
    for (int u = threadIdx.x; u < n_rows * dim; u += blockDim.x) {
        const int r = u / dim, d = u % dim;
        q_rows[r * dim + d] = to_f32(q[(long)(first_token + r / n_heads_here) * ld_q + (long)(first_head + r % n_heads_here) * dim + d]);
    }

    // A block of 32 keys and values comes in 16-byte vectors, up to MAXV of each per thread; which
    // (key, column) a thread's vectors are is fixed for the kernel, so no division is left in the loop.
    constexpr int VEC = 16 / (int)sizeof(T);
    constexpr int MAXV = TILE_KEYS * SIZE / VEC / (TILE_WARPS * 32);
    uint4 key_vec[MAXV], value_vec[MAXV];
    int key_row[MAXV], key_col[MAXV], value_row[MAXV], value_col[MAXV];
#pragma unroll
    for (int i = 0; i < MAXV; i++) {
        const int u = threadIdx.x + i * TILE_WARPS * 32;
        key_row[i] = u < TILE_KEYS * (dim / VEC) ? u / (dim / VEC) : -1;
        key_col[i] = (u % (dim / VEC)) * VEC;
        value_row[i] = u < TILE_KEYS * (vdim / VEC) ? u / (vdim / VEC) : -1;
        value_col[i] = (u % (vdim / VEC)) * VEC;
        key_vec[i] = value_vec[i] = make_uint4(0, 0, 0, 0);
    }
    const int page_shift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;
    auto fetch = [&](const int* bt, int base, int p_last, int p_lo) {
#pragma unroll
        for (int i = 0; i < MAXV; i++) {
            const int kp = base + key_row[i], vp = base + value_row[i];
            if (key_row[i] >= 0 && kp <= p_last && kp >= p_lo) {
                const int block = page_shift >= 0 ? kp >> page_shift : kp / page_size;
                const long slot = (long)bt[block] * page_size + (kp - block * page_size);
                key_vec[i] = *reinterpret_cast<const uint4*>(k_pages + (slot * n_kv_heads + hk) * dim + key_col[i]);
            }
            if (value_row[i] >= 0 && vp <= p_last && vp >= p_lo) {
                const int block = page_shift >= 0 ? vp >> page_shift : vp / page_size;
                const long slot = (long)bt[block] * page_size + (vp - block * page_size);
                value_vec[i] = *reinterpret_cast<const uint4*>(v_pages + (slot * n_kv_heads + hk) * vdim + value_col[i]);
            }
        }
    };

    float* my_weights = weights + warp * TILE_KEYS * R;
    int run_first = 0;
    while (run_first < n_tok) {
        // a run: consecutive tokens of the tile that belong to one request
        const int item = token_item[first_token + run_first];
        int run_last = run_first;
        while (run_last + 1 < n_tok && token_item[first_token + run_last + 1] == item) run_last++;
        const int p_first = positions[first_token + run_first], p_last = positions[first_token + run_last];
        const int lo = first_visible(p_first, window, chunk);
        const int* bt = block_table + (long)item * max_blocks;
        const int first_base = (lo / TILE_KEYS) * TILE_KEYS;
        fetch(bt, first_base, p_last, lo);          // (pages before the first visible key may be gone)
        for (int base = first_base; base <= p_last; base += TILE_KEYS) {
            __syncthreads();                                  // the block before has been read; q_rows are written
            const int n_keys = min(TILE_KEYS, p_last + 1 - base);
#pragma unroll
            for (int i = 0; i < MAXV; i++) {
                if (key_row[i] >= 0 && key_row[i] < n_keys) widen<T>(key_vec[i], keys + key_row[i] * kd + key_col[i]);
                if (value_row[i] >= 0 && value_row[i] < n_keys) widen<T>(value_vec[i], values + value_row[i] * vdim + value_col[i]);
            }
            __syncthreads();
            // the next block's rows are asked for now and arrive while this one is worked on
            if (base + TILE_KEYS <= p_last) fetch(bt, base + TILE_KEYS, p_last, lo);
            // which of the warp's rows see a key of this block at all
            bool any = false, seen[R];
            int first_seen[R];
#pragma unroll
            for (int s = 0; s < R; s++) {
                first_seen[s] = first_visible(row_pos[s], window, chunk);
                seen[s] = row_item[s] == item && base <= row_pos[s] && base + TILE_KEYS > first_seen[s];
                any = any || seen[s];
            }
            if (!any) continue;                               // (uniform in the warp; the barriers are at the loop's head)
            // scores: this lane's key against the warp's rows, four entries at a time
            float dot[R];
#pragma unroll
            for (int s = 0; s < R; s++) dot[s] = 0.0f;
            const float* kr = keys + lane * kd;
#pragma unroll 2
            for (int d = 0; d < dim; d += 4) {
                const float4 b = *reinterpret_cast<const float4*>(kr + d);
#pragma unroll
                for (int s = 0; s < R; s++) {
                    const float4 a = *reinterpret_cast<const float4*>(q_rows + (warp + s * TILE_WARPS) * dim + d);
                    dot[s] = fmaf(a.x, b.x, dot[s]);
                    dot[s] = fmaf(a.y, b.y, dot[s]);
                    dot[s] = fmaf(a.z, b.z, dot[s]);
                    dot[s] = fmaf(a.w, b.w, dot[s]);
                }
            }
            const int pos = base + lane;
#pragma unroll
            for (int s = 0; s < R; s++) {
                const bool mine = seen[s] && lane < n_keys && pos <= row_pos[s] && pos >= first_seen[s];
                const float score = mine ? capped(dot[s] * scale, cap, inv_cap) : -INFINITY;
                const float block_max = warp_max(score);
                float rescale = 1.0f, e = 0.0f;
                if (block_max != -INFINITY) {
                    const float m_new = fmaxf(m[s], block_max);
                    rescale = expf(m[s] - m_new);
                    e = mine ? expf(score - m_new) : 0.0f;
                    m[s] = m_new;
                }
                l[s] = l[s] * rescale + warp_sum(e);
#pragma unroll
                for (int i = 0; i < VPL; i++) acc[s][i] *= rescale;
                my_weights[lane * R + s] = e;
            }
            __syncwarp();
#pragma unroll 4
            for (int j = 0; j < n_keys; j++) {
                float w[R];
#pragma unroll
                for (int s = 0; s < R; s += 2) {
                    const float2 pair = *reinterpret_cast<const float2*>(my_weights + j * R + s);
                    w[s] = pair.x, w[s + 1] = pair.y;
                }
                const float* vr = values + j * vdim;
#pragma unroll
                for (int i = 0; i < VPL; i++) {
                    const int d = lane + 32 * i;
                    if (i + 1 < VPL || d < vdim) {
                        const float v = d < vdim ? vr[d] : 0.0f;
#pragma unroll
                        for (int s = 0; s < R; s++) acc[s][i] = fmaf(w[s], v, acc[s][i]);
                    }
                }
            }
            __syncwarp();
        }
        run_first = run_last + 1;
    }
#pragma unroll
    for (int s = 0; s < R; s++) {
        const int r = warp + s * TILE_WARPS;
        if (r >= n_rows) continue;
        const int token = first_token + r / n_heads_here, head = first_head + r % n_heads_here;
        float sum = l[s], shrink = 1.0f;
        if (sink != nullptr) {
            // the sink's term joins the denominator; the sums are rescaled if it is the largest
            const float top = fmaxf(m[s], sink[head]);
            shrink = expf(m[s] - top);
            sum = sum * shrink + expf(sink[head] - top);
        }
        const float inv = (gate != nullptr ? sigmoid_f(gate[(long)token * ld_gate + head]) : 1.0f) * shrink / sum;
#pragma unroll
        for (int i = 0; i < VPL; i++) {
            const int d = lane + 32 * i;
            if (d < vdim) out[(long)token * ld_out + (long)head * vdim + d] = from_f32<T>(acc[s][i] * inv);
        }
    }
}

// ---------------------------------------------------------------------------
// The same attention as register tiles, for the common sizes (values of 64 or 128 entries, keys of up to 128,
// no gate, no mask of blocks).  A block of 256 threads takes 64 (token, head) rows of one key/value head and walks
// the keys 64 at a time.  Thread (ty, tx) of a 16 x 16 grid holds the scores of rows 4 ty .. 4 ty + 3 against keys
// tx, tx + 16, tx + 32, tx + 48 (sixteen sums, fed by 16-byte reads of q and k rows along the head: eight FMAs a
// read), then, after the block's softmax step, the sums of those rows' values for columns 4 tx .. 4 tx + 3 (and
// 64 + 4 tx .. for values of 128): again sixteen (thirty-two) sums fed by 16-byte reads of the weights' rows and
// of the values' rows.  The sixteen threads of a row lie in one half of a warp: a row's maximum and sum are four
// shuffles, and its weights pass through shared memory between threads of one warp.  Scores, maxima, sums and
// weights are 32-bit.  Tokens of several requests in a tile are taken request by request, as in the kernel above.
// ---------------------------------------------------------------------------
constexpr int BLOCK_ROWS = 64, BLOCK_KEYS = 64;
constexpr int BLOCK_RT = 4;                                   // rows a thread (eight measured slower: 255 registers, one block fewer an SM)
constexpr int BLOCK_THREADS = 16 * BLOCK_ROWS / BLOCK_RT;

template <typename T, int VG>          // VG: 64-entry groups of a value (1 or 2)
__global__ void __launch_bounds__(BLOCK_THREADS)
capped_attention_block_kernel(T* __restrict__ out, long ld_out, const T* __restrict__ q, long ld_q,
                              const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                              const int* __restrict__ block_table, int max_blocks, const int* __restrict__ positions,
                              const int* __restrict__ token_item, int n_tokens, int n_heads, int n_kv_heads, int dim,
                              int page_size, float scale, float cap, int window, const float* __restrict__ sink,
                              int tokens_per_block, int heads_per_block) {
    dependents_may_start();
    wait_for_earlier_kernels();
    constexpr int VDIM = 64 * VG;
    extern __shared__ float shared[];
    const int kd = dim + 4, vd = VDIM + 4, pd = BLOCK_KEYS + 4;
    float* q_rows = shared;                                  // [64][kd]
    float* keys = q_rows + BLOCK_ROWS * kd;                  // [64][kd]
    float* values = keys + BLOCK_KEYS * kd;                  // [64][vd]
    float* weights = values + BLOCK_KEYS * vd;               // [64][pd]
    int* row_pos = reinterpret_cast<int*>(weights + BLOCK_ROWS * pd);     // [64]
    int* row_item = row_pos + BLOCK_ROWS;                    // [64]
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int group = n_heads / n_kv_heads;
    const int chunks = (group + heads_per_block - 1) / heads_per_block;
    const int hk = blockIdx.y / chunks;
    const int first_head = hk * group + (blockIdx.y % chunks) * heads_per_block;
    const int n_heads_here = min(heads_per_block, hk * group + group - first_head);
    // the step's last tokens first: within a request they see the most keys, and a long block that starts last would
    // leave the other SMs idle at the end
    const int first_token = (gridDim.x - 1 - blockIdx.x) * tokens_per_block;
    const int n_tok = min(tokens_per_block, n_tokens - first_token);
    const int n_rows = n_tok * n_heads_here;
    const float inv_cap = cap > 0.0f ? 1.0f / cap : 0.0f;
    constexpr int VEC = 16 / (int)sizeof(T);

    for (int r = tid; r < BLOCK_ROWS; r += blockDim.x) {
        const bool live = r < n_rows;
        const int token = live ? first_token + r / n_heads_here : 0;
        row_pos[r] = live ? positions[token] : -1;
        row_item[r] = live ? token_item[token] : -1;
    }
    for (int u = tid; u < BLOCK_ROWS * (dim / VEC); u += blockDim.x) {
        const int r = u / (dim / VEC), d = (u % (dim / VEC)) * VEC;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < n_rows)
            v = *reinterpret_cast<const uint4*>(q + (long)(first_token + r / n_heads_here) * ld_q + (long)(first_head + r % n_heads_here) * dim + d);
        widen<T>(v, q_rows + r * kd + d);
    }
    __syncthreads();
    constexpr int RT = BLOCK_RT;
    int my_pos[RT], my_item[RT], my_first[RT];
    float m[RT], l[RT], o[RT][4 * VG];
#pragma unroll
    for (int i = 0; i < RT; i++) {
        my_pos[i] = row_pos[ty * RT + i], my_item[i] = row_item[ty * RT + i];
        my_first[i] = first_visible(my_pos[i], window, 0);
        m[i] = -INFINITY, l[i] = 0.0f;
#pragma unroll
        for (int c = 0; c < 4 * VG; c++) o[i][c] = 0.0f;
    }
    const int page_shift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;
    // A tile of 64 keys and values comes in 16-byte vectors, a fixed few of each per thread, asked for a tile ahead;
    // which (key, column) a thread's vectors are is fixed for the kernel.
    constexpr int MAXK = BLOCK_KEYS * 128 / VEC / BLOCK_THREADS, MAXV = BLOCK_KEYS * VDIM / VEC / BLOCK_THREADS;
    uint4 key_vec[MAXK], value_vec[MAXV];
    int key_row[MAXK], key_col[MAXK], value_row[MAXV], value_col[MAXV];
#pragma unroll
    for (int i = 0; i < MAXK; i++) {
        const int u = tid + i * BLOCK_THREADS;
        key_row[i] = u < BLOCK_KEYS * (dim / VEC) ? u / (dim / VEC) : -1;
        key_col[i] = (u % (dim / VEC)) * VEC;
        key_vec[i] = make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int i = 0; i < MAXV; i++) {
        const int u = tid + i * BLOCK_THREADS;
        value_row[i] = u / (VDIM / VEC);
        value_col[i] = (u % (VDIM / VEC)) * VEC;
        value_vec[i] = make_uint4(0u, 0u, 0u, 0u);
    }
    auto fetch = [&](const int* bt, int base, int p_last, int p_lo) {
#pragma unroll
        for (int i = 0; i < MAXK; i++) {
            const int kp = base + key_row[i];
            key_vec[i] = make_uint4(0u, 0u, 0u, 0u);
            if (key_row[i] >= 0 && kp <= p_last && kp >= p_lo) {          // (pages before the first visible key may be gone)
                const int block = page_shift >= 0 ? kp >> page_shift : kp / page_size;
                const long slot = (long)bt[block] * page_size + (kp - block * page_size);
                key_vec[i] = *reinterpret_cast<const uint4*>(k_pages + (slot * n_kv_heads + hk) * dim + key_col[i]);
            }
        }
#pragma unroll
        for (int i = 0; i < MAXV; i++) {
            const int vp = base + value_row[i];
            value_vec[i] = make_uint4(0u, 0u, 0u, 0u);
            if (vp <= p_last && vp >= p_lo) {
                const int block = page_shift >= 0 ? vp >> page_shift : vp / page_size;
                const long slot = (long)bt[block] * page_size + (vp - block * page_size);
                value_vec[i] = *reinterpret_cast<const uint4*>(v_pages + (slot * n_kv_heads + hk) * VDIM + value_col[i]);
            }
        }
    };

    int run_first = 0;
    while (run_first < n_tok) {
        const int item = token_item[first_token + run_first];
        int run_last = run_first;
        while (run_last + 1 < n_tok && token_item[first_token + run_last + 1] == item) run_last++;
        const int p_first = positions[first_token + run_first], p_last = positions[first_token + run_last];
        const int lo = first_visible(p_first, window, 0);
        const int* bt = block_table + (long)item * max_blocks;
        const int first_base = (lo / BLOCK_KEYS) * BLOCK_KEYS;
        fetch(bt, first_base, p_last, lo);
        for (int base = first_base; base <= p_last; base += BLOCK_KEYS) {
            __syncthreads();                                  // the tile before has been read
#pragma unroll
            for (int i = 0; i < MAXK; i++)
                if (key_row[i] >= 0) widen<T>(key_vec[i], keys + key_row[i] * kd + key_col[i]);
#pragma unroll
            for (int i = 0; i < MAXV; i++) widen<T>(value_vec[i], values + value_row[i] * vd + value_col[i]);
            __syncthreads();
            // the next tile's rows are asked for now and arrive while this one is worked on
            if (base + BLOCK_KEYS <= p_last) fetch(bt, base + BLOCK_KEYS, p_last, lo);
            // does any row of this warp see a key of this tile?
            bool any = false;
#pragma unroll
            for (int i = 0; i < RT; i++)
                any = any || (my_item[i] == item && base <= my_pos[i] && base + BLOCK_KEYS > my_first[i]);
            if (!__any_sync(0xffffffffu, any)) continue;      // (uniform in the warp; the barriers are at the loop's head)
            float acc[RT][4];
#pragma unroll
            for (int i = 0; i < RT; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;
#pragma unroll 2
            for (int d = 0; d < dim; d += 4) {
                float4 a[RT], b[4];
#pragma unroll
                for (int i = 0; i < RT; i++) a[i] = *reinterpret_cast<const float4*>(q_rows + (ty * RT + i) * kd + d);
#pragma unroll
                for (int j = 0; j < 4; j++) b[j] = *reinterpret_cast<const float4*>(keys + (tx + 16 * j) * kd + d);
#pragma unroll
                for (int i = 0; i < RT; i++)
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        acc[i][j] = fmaf(a[i].x, b[j].x, acc[i][j]);
                        acc[i][j] = fmaf(a[i].y, b[j].y, acc[i][j]);
                        acc[i][j] = fmaf(a[i].z, b[j].z, acc[i][j]);
                        acc[i][j] = fmaf(a[i].w, b[j].w, acc[i][j]);
                    }
            }
#pragma unroll
            for (int i = 0; i < RT; i++) {
                const bool row_here = my_item[i] == item;
                float score[4], top = -INFINITY;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int pos = base + tx + 16 * j;
                    const bool seen = row_here && pos <= my_pos[i] && pos >= my_first[i];
                    score[j] = seen ? capped(acc[i][j] * scale, cap, inv_cap) : -INFINITY;
                    top = fmaxf(top, score[j]);
                }
#pragma unroll
                for (int step = 8; step > 0; step >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, step));
                float rescale = 1.0f, e[4] = {0.0f, 0.0f, 0.0f, 0.0f}, sum = 0.0f;
                if (top != -INFINITY) {
                    const float m_new = fmaxf(m[i], top);
                    rescale = expf(m[i] - m_new);
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        e[j] = score[j] == -INFINITY ? 0.0f : expf(score[j] - m_new);
                        sum += e[j];
                    }
                    m[i] = m_new;
                }
#pragma unroll
                for (int step = 8; step > 0; step >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, step);
                l[i] = l[i] * rescale + sum;
#pragma unroll
                for (int c = 0; c < 4 * VG; c++) o[i][c] *= rescale;
#pragma unroll
                for (int j = 0; j < 4; j++) weights[(ty * RT + i) * pd + tx + 16 * j] = e[j];
            }
            __syncwarp();                                     // a row's sixteen threads lie in this warp
#pragma unroll 2
            for (int j = 0; j < BLOCK_KEYS; j += 4) {
                float4 w[RT];
#pragma unroll
                for (int i = 0; i < RT; i++) w[i] = *reinterpret_cast<const float4*>(weights + (ty * RT + i) * pd + j);
#pragma unroll
                for (int jj = 0; jj < 4; jj++) {
#pragma unroll
                    for (int g = 0; g < VG; g++) {
                        const float4 v = *reinterpret_cast<const float4*>(values + (j + jj) * vd + 64 * g + tx * 4);
#pragma unroll
                        for (int i = 0; i < RT; i++) {
                            const float p = jj == 0 ? w[i].x : (jj == 1 ? w[i].y : (jj == 2 ? w[i].z : w[i].w));
                            o[i][4 * g] = fmaf(p, v.x, o[i][4 * g]);
                            o[i][4 * g + 1] = fmaf(p, v.y, o[i][4 * g + 1]);
                            o[i][4 * g + 2] = fmaf(p, v.z, o[i][4 * g + 2]);
                            o[i][4 * g + 3] = fmaf(p, v.w, o[i][4 * g + 3]);
                        }
                    }
                }
            }
            __syncwarp();                                     // the weights are read before the next tile's are written
        }
        run_first = run_last + 1;
    }
#pragma unroll
    for (int i = 0; i < RT; i++) {
        const int r = ty * RT + i;
        if (r >= n_rows) continue;
        const int token = first_token + r / n_heads_here, head = first_head + r % n_heads_here;
        float sum = l[i], shrink = 1.0f;
        if (sink != nullptr) {
            const float top = fmaxf(m[i], sink[head]);
            shrink = expf(m[i] - top);
            sum = sum * shrink + expf(sink[head] - top);
        }
        const float inv = shrink / sum;
#pragma unroll
        for (int g = 0; g < VG; g++)
#pragma unroll
            for (int c = 0; c < 4; c++)
                out[(long)token * ld_out + (long)head * VDIM + 64 * g + tx * 4 + c] = from_f32<T>(o[i][4 * g + c] * inv);
    }
}

static size_t capped_block_shared(int dim, int vdim) {
    return sizeof(float) * ((size_t)2 * BLOCK_ROWS * (dim + 4) + (size_t)BLOCK_KEYS * (vdim + 4) + (size_t)BLOCK_ROWS * (BLOCK_KEYS + 4)) +
           sizeof(int) * 2 * BLOCK_ROWS;
}

// (keys in whole 16-byte vectors, values of 64 or 128 entries)
static bool capped_block_takes(int dim, int vdim, int vec) {
    return dim > 0 && dim <= 128 && dim % vec == 0 && dim % 4 == 0 && (vdim == 64 || vdim == 128);
}

template <typename T, int VG>
static int launch_capped_block(void* out, long ld_out, const void* q, long ld_q, const void* k_pages, const void* v_pages,
                               const int* block_table, int max_blocks, const int* positions, const int* token_item, int n_tokens,
                               int n_heads, int n_kv_heads, int dim, int page_size, float scale, float cap, int window,
                               const float* sink, cudaStream_t s) {
    const int group = n_heads / n_kv_heads;
    const int heads_per_block = group < BLOCK_ROWS ? group : BLOCK_ROWS;
    const int tokens_per_block = BLOCK_ROWS / heads_per_block;
    const int chunks = (group + heads_per_block - 1) / heads_per_block;
    const size_t shared = capped_block_shared(dim, 64 * VG);
    cudaError_t e = cudaFuncSetAttribute(capped_attention_block_kernel<T, VG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    if (e != cudaSuccess) return fail("capped_attention: the register tiles' shared memory was refused");
    cudaFuncSetAttribute(capped_attention_block_kernel<T, VG>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    dim3 grid((n_tokens + tokens_per_block - 1) / tokens_per_block, n_kv_heads * chunks);
    launch_kernel(g_dependent_launch != 0, capped_attention_block_kernel<T, VG>, grid, dim3(BLOCK_THREADS), shared, s, (T*)out, ld_out, (const T*)q,
                  ld_q, (const T*)k_pages, (const T*)v_pages, block_table, max_blocks, positions, token_item, n_tokens, n_heads,
                  n_kv_heads, dim, page_size, scale, cap, window, sink, tokens_per_block, heads_per_block);
    return check_launch("capped_attention_block_kernel");
}

static size_t capped_tiled_shared(int dim, int vdim, int rows_per_warp) {
    return sizeof(float) * ((size_t)TILE_WARPS * rows_per_warp * dim + (size_t)TILE_KEYS * (dim + 4) + (size_t)TILE_KEYS * vdim +
                            (size_t)TILE_WARPS * TILE_KEYS * rows_per_warp);
}

// (keys and values in whole 16-byte vectors: sizes that are multiples of `vec` elements)
extern "C" int mllm_hybrid_capped_attention_tiled_takes(int dim, int vdim, int vec) {
    return dim > 0 && vdim > 0 && dim % vec == 0 && vdim % vec == 0 && dim % 4 == 0 && vdim % 4 == 0 && dim <= CAP_MAX_HEAD &&
           vdim <= CAP_MAX_HEAD && capped_tiled_shared(dim, vdim, 2) <= 160 * 1024;
}

template <typename T, int R, int SIZE>
static int launch_capped_tiles(void* out, long ld_out, const void* q, long ld_q, const void* k_pages, const void* v_pages,
                               const int* block_table, int max_blocks, const int* positions, const int* token_item, int n_tokens,
                               int n_heads, int n_kv_heads, int dim, int vdim, int page_size, float scale, float cap, int window,
                               int chunk, const float* gate, long ld_gate, const float* sink, cudaStream_t s) {
    constexpr int ROWS = TILE_WARPS * R;
    const int group = n_heads / n_kv_heads;
    const int heads_per_block = group < ROWS ? group : ROWS;
    const int tokens_per_block = ROWS / heads_per_block;
    const int chunks = (group + heads_per_block - 1) / heads_per_block;
    const size_t shared = capped_tiled_shared(dim, vdim, R);
    cudaError_t e = cudaFuncSetAttribute(capped_attention_tiled_kernel<T, R, SIZE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    if (e != cudaSuccess) return fail("capped_attention: the tiles' shared memory was refused");
    // several blocks an SM: as much of the SM's memory as shared memory as they need
    cudaFuncSetAttribute(capped_attention_tiled_kernel<T, R, SIZE>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    dim3 grid((n_tokens + tokens_per_block - 1) / tokens_per_block, n_kv_heads * chunks);
    launch_kernel(g_dependent_launch != 0, capped_attention_tiled_kernel<T, R, SIZE>, grid, dim3(TILE_WARPS * 32), shared, s, (T*)out,
                  ld_out, (const T*)q, ld_q, (const T*)k_pages, (const T*)v_pages, block_table, max_blocks, positions, token_item,
                  n_tokens, n_heads, n_kv_heads, dim, vdim, page_size, scale, cap, window, chunk, gate, ld_gate, sink,
                  tokens_per_block, heads_per_block);
    return check_launch("capped_attention_tiled_kernel");
}

template <typename T>
static int launch_capped_attention(bool tiled, void* out, long ld_out, const void* q, long ld_q, const void* k_pages,
                                   const void* v_pages, const int* block_table, int max_blocks, const int* positions,
                                   const int* token_item, int n_tokens, int n_heads, int n_kv_heads, int dim, int vdim,
                                   int page_size, float scale, float cap, int window, int chunk, const float* gate, long ld_gate,
                                   const float* sink, cudaStream_t s) {
    if (!tiled) {
        launch_kernel(g_dependent_launch != 0, capped_attention_plain_kernel<T>, dim3(n_tokens, n_heads), dim3(128), 0, s, (T*)out,
                      ld_out, (const T*)q, ld_q, (const T*)k_pages, (const T*)v_pages, block_table, max_blocks, positions,
                      token_item, n_heads, n_kv_heads, dim, vdim, page_size, scale, cap, window, chunk, gate, ld_gate, sink);
        return check_launch("capped_attention_plain_kernel");
    }
    // the common sizes go to the register tiles
    if (gate == nullptr && chunk == 0 && n_tokens * (long)n_heads >= 2048 && capped_block_takes(dim, vdim, 16 / (int)sizeof(T)) &&
        (ld_q * sizeof(T)) % 16 == 0) {
        if (vdim == 64)
            return launch_capped_block<T, 1>(out, ld_out, q, ld_q, k_pages, v_pages, block_table, max_blocks, positions, token_item,
                                             n_tokens, n_heads, n_kv_heads, dim, page_size, scale, cap, window, sink, s);
        return launch_capped_block<T, 2>(out, ld_out, q, ld_q, k_pages, v_pages, block_table, max_blocks, positions, token_item,
                                         n_tokens, n_heads, n_kv_heads, dim, page_size, scale, cap, window, sink, s);
    }
    // rows a warp: four where the step has rows enough for the blocks to fill the GPU all the same
    // (and their shared memory fits), else two
    const long rows = (long)n_tokens * n_heads;
    int per_warp = rows >= 8192 ? 4 : 2;
    if (capped_tiled_shared(dim, vdim, per_warp) > 160 * 1024) per_warp = 2;
#define TILES(R, SIZE)                                                                                                        \
    return launch_capped_tiles<T, R, SIZE>(out, ld_out, q, ld_q, k_pages, v_pages, block_table, max_blocks, positions, token_item, \
                                           n_tokens, n_heads, n_kv_heads, dim, vdim, page_size, scale, cap, window, chunk, gate, ld_gate, sink, s)
    const int size = (dim > vdim ? dim : vdim) <= 64 ? 64 : ((dim > vdim ? dim : vdim) <= 128 ? 128 : 256);
    if (per_warp == 4) { if (size == 64) TILES(4, 64); if (size == 128) TILES(4, 128); TILES(4, 256); }
    if (size == 64) TILES(2, 64);
    if (size == 128) TILES(2, 128);
    TILES(2, 256);
#undef TILES
}

extern "C" int mllm_hybrid_capped_attention(void* out, long ld_out, const void* q, long ld_q, const void* k_pages,
                                            const void* v_pages, const int* block_table, int max_blocks, const int* positions,
                                            const int* token_item, int n_tokens, int n_heads, int n_kv_heads, int dim, int vdim,
                                            int page_size, float scale, float cap, int window, int chunk, const float* gate,
                                            long ld_gate, const float* sink, int tiled, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (dim <= 0 || dim > CAP_MAX_HEAD || vdim <= 0 || vdim > CAP_MAX_HEAD) return fail("capped_attention: key and value sizes must be in 1..256");
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0) return fail("capped_attention: heads must be a multiple of the key/value heads");
    if (n_heads > 65535) return fail("capped_attention: too many heads for one launch");
    if (tiled && !mllm_hybrid_capped_attention_tiled_takes(dim, vdim, dtype == DT_F32 ? 4 : 8)) return fail("capped_attention: the tiles do not take these sizes");
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == DT_F32)
        return launch_capped_attention<float>(tiled != 0, out, ld_out, q, ld_q, k_pages, v_pages, block_table, max_blocks, positions,
                                              token_item, n_tokens, n_heads, n_kv_heads, dim, vdim, page_size, scale, cap, window, chunk, gate,
                                              ld_gate, sink, s);
    if (dtype == DT_BF16)
        return launch_capped_attention<bf16>(tiled != 0, out, ld_out, q, ld_q, k_pages, v_pages, block_table, max_blocks, positions,
                                             token_item, n_tokens, n_heads, n_kv_heads, dim, vdim, page_size, scale, cap, window, chunk, gate,
                                             ld_gate, sink, s);
    return fail("capped_attention: unknown dtype");
}

// ---------------------------------------------------------------------------
// Linear recurrence with a matrix state per head, S [dim, vdim] in 32-bit:
//   a_t = exp(-exp(log_rate[h]) * step_t),  step_t = softplus(gate_a[t, h] + step_bias[h])
//   state-space form:  b_t = step_t;               u_t = b_t v_t
//   delta rule:        b_t = sigmoid(gate_b[t, h]); u_t = b_t (v_t - (a_t S)^T k_t)
//   S <- a_t S + k_t u_t^T;   out_t = S^T q_t (+ skip[h] v_t)
// Query/key head of head h: h / (heads / qk_heads).  With unit_norm, q and k are divided by
// sqrt(sum(x^2) + 1e-6) per head first; q is multiplied by q_scale.
// With channel_decay the decay is one per key channel instead: gate_a [T, heads * dim] and step_bias
// [heads * dim], a_t[i] = exp(-exp(log_rate[h]) * softplus(gate_a[t, h, i] + step_bias[h, i])), and row i of S
// is multiplied by a_t[i] before the old column is read: S <- diag(a_t) S; u_t = b_t (v_t - S^T k_t);
// S <- S + k_t u_t^T.
// One block per (entry, head, slice of the value entries): a column of S belongs to LANES threads
// of one warp, each with DPT rows in registers; both sums over the old column (with k and with q)
// are taken in one pass, and the read-out follows from them: S_new^T q = a S^T q + u (k . q).
// The entry's tokens are taken in order, TOK at a time through shared memory; a chunk's rows are
// asked for into registers while the chunk before it is worked on.
// ---------------------------------------------------------------------------
struct RecurrenceParams {
    float* out; long ld_out;
    const void* q; const void* k; const void* v; long ld_q, ld_k, ld_v;
    const float* gate_a; const float* gate_b; long ld_gate_a, ld_gate_b;
    const float* log_rate; const float* step_bias; const float* skip;
    float* state; long state_stride;
    const int* item_slot; const int* item_offset; const int* item_count;
    int heads, qk_heads, dim, vdim;
    float q_scale;
    int delta, unit_norm, writes;
    int channel_decay;
};

template <typename T, int DPT, int LANES, int TOK, int CPT, bool CHANNEL>      // CPT: columns of the state a thread takes
__global__ void __launch_bounds__(128) linear_recurrence_kernel(RecurrenceParams pp) {
    dependents_may_start();
    wait_for_earlier_kernels();
    constexpr int GROUPS = 128 / LANES;                    // groups of lanes; each takes CPT columns of the state,
    constexpr int COLS = GROUPS * CPT;                     // GROUPS apart, whose chains of sums run side by side
    constexpr int PAD = DPT + 4;                           // a lane's DPT entries of a staged row, 16 bytes apart from the
    constexpr int ROW = LANES * PAD;                       // next lane's in the banks: four entries are read at a time
    constexpr int TPR = 128 / (2 * TOK);                   // threads that bring one staged row (k or q of a token)
    constexpr int PER = (DPT * LANES + TPR - 1) / TPR;     // entries of that row a thread brings
    constexpr int VPER = (TOK * COLS + 127) / 128;         // values a thread brings
    extern __shared__ float shared[];
    const int dim = pp.dim, vdim = pp.vdim;
    float* ks = shared;                         // [TOK][ROW]: entry i of a row at (i / DPT) * PAD + i % DPT, zero past dim
    float* qs = ks + TOK * ROW;                 // [TOK][ROW]
    float* vs = qs + TOK * ROW;                 // [TOK][COLS]
    float* as = vs + TOK * COLS;                // [TOK] the step's gate, then the decay
    float* bs = as + TOK;                       // [TOK] the write gate, then the write strength
    float* kq = bs + TOK;                       // [TOK] k . q
    float* gs = kq + TOK;                       // [TOK][ROW] (CHANNEL only): the decay of every key channel, laid out as ks
    constexpr int GPER = CHANNEL ? (TOK * DPT * LANES + 127) / 128 : 1;     // decays a thread brings
    const int item = blockIdx.x, head = blockIdx.y;
    const int count = pp.item_count[item];
    if (count <= 0) return;
    const long first = pp.item_offset[item];
    const int qk_head = head / (pp.heads / pp.qk_heads);
    const int lane_in = threadIdx.x % LANES, col_local = threadIdx.x / LANES;
    // this thread's columns: col_local, col_local + GROUPS, ... of the block's COLS
    // this thread's part of its column of the state: rows lane_in * DPT .. + DPT - 1 (zero past dim, and it stays zero)
    float* S = pp.state + (long)pp.item_slot[item] * pp.state_stride + (long)head * dim * vdim;
    // (the block's slice of the state goes through shared memory both ways, so that the global
    // reads and writes run along the rows of S, whatever the lanes' share of a column is)
    float s[CPT][DPT];
    for (int u = threadIdx.x; u < dim * COLS; u += 128) {
        const int i = u / COLS, c = blockIdx.z * COLS + u % COLS;
        shared[u] = c < vdim ? S[(long)i * vdim + c] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < DPT; r++) {
        const int i = lane_in * DPT + r;
#pragma unroll
        for (int c = 0; c < CPT; c++) s[c][r] = i < dim ? shared[i * COLS + col_local + c * GROUPS] : 0.0f;
    }
    __syncthreads();
    const float rate = expf(pp.log_rate[head]);
    const float bias = CHANNEL ? 0.0f : pp.step_bias[head];
    const float skip = pp.skip != nullptr ? pp.skip[head] : 0.0f;
    const T* q = (const T*)pp.q;
    const T* k = (const T*)pp.k;
    const T* v = (const T*)pp.v;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // What a thread brings of every chunk of TOK tokens: PER entries of one row (the k or the q of one
    // token), VPER values, and (the first threads) a token's gates.  The next chunk is asked for
    // before the current one is worked on, so its way through the memory lies under the sums.
    const int row = threadIdx.x / TPR, row_sub = threadIdx.x % TPR;
    const int row_token = row >> 1;
    const T* row_base = (row & 1) ? q : k;
    const long row_ld = (row & 1) ? pp.ld_q : pp.ld_k;
    float* row_smem = ((row & 1) ? qs : ks) + row_token * ROW;
    T raw[PER], raw_v[VPER];
    float raw_a = 0.0f, raw_b = 0.0f;
    float raw_g[GPER];
    // (the channel's bias is the same in every chunk: it is read once here, and added when the chunk is staged,
    // so that asking for a chunk waits for nothing)
    float bias_g[GPER];
    if (CHANNEL) {
#pragma unroll
        for (int i = 0; i < GPER; i++) {
            const int d = (threadIdx.x + 128 * i) % (DPT * LANES);
            bias_g[i] = d < dim ? pp.step_bias[(long)head * dim + d] : 0.0f;
        }
    }
    auto ask = [&](int start) {
        const int n = min(TOK, count - start);
        const long t0 = first + start;
#pragma unroll
        for (int i = 0; i < PER; i++) {
            const int d = row_sub + TPR * i;
            raw[i] = (row_token < n && d < dim) ? row_base[(t0 + row_token) * row_ld + (long)qk_head * dim + d] : from_f32<T>(0.0f);
        }
#pragma unroll
        for (int i = 0; i < VPER; i++) {
            const int u = threadIdx.x + 128 * i, tt = u / COLS, c = blockIdx.z * COLS + u % COLS;
            raw_v[i] = (tt < n && c < vdim) ? v[(t0 + tt) * pp.ld_v + (long)head * vdim + c] : from_f32<T>(0.0f);
        }
        if (threadIdx.x < n) {
            if (!CHANNEL) raw_a = pp.gate_a[(t0 + threadIdx.x) * pp.ld_gate_a + head];
            if (pp.delta) raw_b = pp.gate_b[(t0 + threadIdx.x) * pp.ld_gate_b + head];
        }
        if (CHANNEL) {
#pragma unroll
            for (int i = 0; i < GPER; i++) {
                const int u = threadIdx.x + 128 * i, tt = u / (DPT * LANES), d = u % (DPT * LANES);
                raw_g[i] = (tt < n && d < dim) ? pp.gate_a[(t0 + tt) * pp.ld_gate_a + (long)head * dim + d] : 0.0f;
            }
        }
    };
    ask(0);
    for (int start = 0; start < count; start += TOK) {
        const int n = min(TOK, count - start);
        __syncthreads();                                      // the chunk before has been read
#pragma unroll
        for (int i = 0; i < PER; i++) {
            const int d = row_sub + TPR * i;
            if (d < DPT * LANES) row_smem[(d / DPT) * PAD + d % DPT] = to_f32(raw[i]);       // (zero past dim)
        }
#pragma unroll
        for (int i = 0; i < VPER; i++) {
            const int u = threadIdx.x + 128 * i;
            if (u < TOK * COLS) vs[u] = to_f32(raw_v[i]);
        }
        if (threadIdx.x < TOK) {
            // a thread a token: the step, the decay, the write strength
            const float step = softplus_f(raw_a + bias);
            as[threadIdx.x] = CHANNEL ? 1.0f : expf(-rate * step);
            bs[threadIdx.x] = pp.delta ? sigmoid_f(raw_b) : step;
        }
        if (CHANNEL) {
#pragma unroll
            for (int i = 0; i < GPER; i++) {
                const int u = threadIdx.x + 128 * i, tt = u / (DPT * LANES), d = u % (DPT * LANES);
                if (tt < TOK) gs[tt * ROW + (d / DPT) * PAD + d % DPT] = expf(-rate * softplus_f(raw_g[i] + bias_g[i]));
            }
        }
        __syncthreads();
        // a warp finishes TOK / 4 tokens: unit vectors if asked, and k . q; the sums of its tokens are
        // taken side by side, so that their exchanges between the lanes lie under one another
        {
            constexpr int MINE = TOK / 4;
            float sk[MINE], sq[MINE], sd[MINE];
#pragma unroll
            for (int j = 0; j < MINE; j++) {
                const int tt = warp + 4 * j;
                sk[j] = sq[j] = sd[j] = 0.0f;
                if (tt < n)
                    for (int d = lane; d < DPT * LANES; d += 32) {
                        const int at = tt * ROW + (d / DPT) * PAD + d % DPT;
                        const float kv = ks[at], qv = qs[at];
                        sk[j] = fmaf(kv, kv, sk[j]), sq[j] = fmaf(qv, qv, sq[j]), sd[j] = fmaf(kv, qv, sd[j]);
                    }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                for (int j = 0; j < MINE; j++) {
                    sk[j] += __shfl_xor_sync(0xffffffffu, sk[j], o);
                    sq[j] += __shfl_xor_sync(0xffffffffu, sq[j], o);
                    sd[j] += __shfl_xor_sync(0xffffffffu, sd[j], o);
                }
#pragma unroll
            for (int j = 0; j < MINE; j++) {
                const int tt = warp + 4 * j;
                if (tt >= n) continue;
                const float fk = pp.unit_norm ? 1.0f / sqrtf(sk[j] + 1e-6f) : 1.0f;
                const float fq = pp.unit_norm ? pp.q_scale / sqrtf(sq[j] + 1e-6f) : pp.q_scale;
                if (pp.unit_norm || fq != 1.0f)
                    for (int d = lane; d < DPT * LANES; d += 32) {
                        const int at = tt * ROW + (d / DPT) * PAD + d % DPT;
                        ks[at] *= fk, qs[at] *= fq;
                    }
                if (lane == 0) kq[tt] = sd[j] * fk * fq;
            }
        }
        __syncthreads();
        if (start + TOK < count) ask(start + TOK);
        for (int tt = 0; tt < n; tt++) {
            const float* kr = ks + tt * ROW + lane_in * PAD;
            const float* qr = qs + tt * ROW + lane_in * PAD;
            float kreg[DPT];
            float dk[CPT][2], dq[CPT][2];                      // two chains each: half the latency
#pragma unroll
            for (int c = 0; c < CPT; c++) dk[c][0] = dk[c][1] = dq[c][0] = dq[c][1] = 0.0f;
#pragma unroll
            for (int r = 0; r < DPT; r += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(kr + r);
                const float4 q4 = *reinterpret_cast<const float4*>(qr + r);
                kreg[r] = k4.x, kreg[r + 1] = k4.y, kreg[r + 2] = k4.z, kreg[r + 3] = k4.w;
                if (CHANNEL) {
                    // every row of the state decays by its own factor first; the sums then read the decayed rows
                    const float4 g4 = *reinterpret_cast<const float4*>(gs + tt * ROW + lane_in * PAD + r);
#pragma unroll
                    for (int c = 0; c < CPT; c++) s[c][r] *= g4.x, s[c][r + 1] *= g4.y, s[c][r + 2] *= g4.z, s[c][r + 3] *= g4.w;
                }
#pragma unroll
                for (int c = 0; c < CPT; c++) {
                    dk[c][0] = fmaf(s[c][r], k4.x, dk[c][0]), dq[c][0] = fmaf(s[c][r], q4.x, dq[c][0]);
                    dk[c][1] = fmaf(s[c][r + 1], k4.y, dk[c][1]), dq[c][1] = fmaf(s[c][r + 1], q4.y, dq[c][1]);
                    dk[c][0] = fmaf(s[c][r + 2], k4.z, dk[c][0]), dq[c][0] = fmaf(s[c][r + 2], q4.z, dq[c][0]);
                    dk[c][1] = fmaf(s[c][r + 3], k4.w, dk[c][1]), dq[c][1] = fmaf(s[c][r + 3], q4.w, dq[c][1]);
                }
            }
            float sum_k[CPT], sum_q[CPT];
#pragma unroll
            for (int c = 0; c < CPT; c++) sum_k[c] = dk[c][0] + dk[c][1], sum_q[c] = dq[c][0] + dq[c][1];
#pragma unroll
            for (int o = LANES / 2; o > 0; o >>= 1)
#pragma unroll
                for (int c = 0; c < CPT; c++) {
                    sum_k[c] += __shfl_xor_sync(0xffffffffu, sum_k[c], o);
                    sum_q[c] += __shfl_xor_sync(0xffffffffu, sum_q[c], o);
                }
            // (with a decay per key channel the rows have decayed already: a factor of one, known when compiled)
            const float a = CHANNEL ? 1.0f : as[tt], b = bs[tt], both = kq[tt];
#pragma unroll
            for (int c = 0; c < CPT; c++) {
                const float value = vs[tt * COLS + col_local + c * GROUPS];
                const float u = pp.delta ? b * (value - a * sum_k[c]) : b * value;
#pragma unroll
                for (int r = 0; r < DPT; r++) s[c][r] = fmaf(kreg[r], u, a * s[c][r]);
                const int col = blockIdx.z * COLS + col_local + c * GROUPS;
                if (col < vdim && lane_in == 0)
                    pp.out[(first + start + tt) * pp.ld_out + (long)head * vdim + col] = fmaf(u, both, a * sum_q[c]) + skip * value;
            }
        }
    }
    if (pp.writes) {
        __syncthreads();
#pragma unroll
        for (int r = 0; r < DPT; r++) {
            const int i = lane_in * DPT + r;
#pragma unroll
            for (int c = 0; c < CPT; c++)
                if (i < dim) shared[i * COLS + col_local + c * GROUPS] = s[c][r];
        }
        __syncthreads();
        for (int u = threadIdx.x; u < dim * COLS; u += 128) {
            const int i = u / COLS, c = blockIdx.z * COLS + u % COLS;
            if (c < vdim) S[(long)i * vdim + c] = shared[u];
        }
    }
}

template <typename T, int DPT, int LANES, int TOK, int CPT, bool CHANNEL>
static int launch_recurrence_as(const RecurrenceParams& pp, int n_items, cudaStream_t s) {
    constexpr int COLS = 128 / LANES * CPT;
    // the staged chunk, or the block's slice of the state on its way in and out, whichever is larger
    const size_t staged = (size_t)(CHANNEL ? 3 : 2) * TOK * LANES * (DPT + 4) + TOK * COLS + 3 * TOK, slice = (size_t)DPT * LANES * COLS;
    const size_t shared = sizeof(float) * (staged > slice ? staged : slice);
    dim3 grid(n_items, pp.heads, (pp.vdim + COLS - 1) / COLS);
    if (shared > 48 * 1024 &&
        cudaFuncSetAttribute(linear_recurrence_kernel<T, DPT, LANES, TOK, CPT, CHANNEL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared) != cudaSuccess)
        return fail("linear_recurrence: the staged rows' shared memory was refused");
    launch_kernel(g_dependent_launch != 0, linear_recurrence_kernel<T, DPT, LANES, TOK, CPT, CHANNEL>, grid, dim3(128), shared, s, pp);
    return check_launch("linear_recurrence_kernel");
}

template <typename T, int DPT, int LANES, int TOK, int CPT>
static int launch_recurrence(const RecurrenceParams& pp, int n_items, cudaStream_t s) {
    if (pp.channel_decay) return launch_recurrence_as<T, DPT, LANES, TOK, CPT, true>(pp, n_items, s);
    return launch_recurrence_as<T, DPT, LANES, TOK, CPT, false>(pp, n_items, s);
}

// A column of the state lies in the registers of 4 to 32 lanes of a warp.  Prompt portions: eight
// rows a lane up to a key size of 256 (short sums).  Steps of few tokens per entry: as many rows a
// lane as registers hold, so that the blocks, each of which pays the same chain of loads for its
// one token, are few.
template <typename T>
static int pick_recurrence(const RecurrenceParams& pp, int n_items, int n_tokens, cudaStream_t s) {
    if (pp.dim <= 32) return launch_recurrence<T, 8, 4, 16, 1>(pp, n_items, s);
    if (n_tokens <= 4 * n_items) {
        if (pp.dim <= 64) return launch_recurrence<T, 16, 4, 16, 1>(pp, n_items, s);
        if (pp.dim <= 128) return launch_recurrence<T, 32, 4, 16, 1>(pp, n_items, s);
    } else if (pp.dim <= 128) {
        // Prompt portions.  The walk from token to token is a chain of dependent sums and exchanges
        // between lanes; a thread takes two columns, whose chains run in one another's gaps, or four
        // where two would leave the busy entries' blocks more than one an SM (entries of a step that
        // is filled up to a round shape may be empty: portions are taken to hold 1,024 tokens).
        // Eight columns a thread measured slower: every column has its own exchanges.
        const int groups = pp.dim <= 64 ? 16 : 8;
        int busy = (n_tokens + 1023) / 1024;
        if (busy > n_items) busy = n_items;
        const bool four = (long)busy * pp.heads * ((pp.vdim + groups * 2 - 1) / (groups * 2)) > 148;
        if (pp.dim <= 64) {
            if (four) return launch_recurrence<T, 8, 8, 16, 4>(pp, n_items, s);
            return launch_recurrence<T, 8, 8, 16, 2>(pp, n_items, s);
        }
        if (four) return launch_recurrence<T, 8, 16, 16, 4>(pp, n_items, s);
        return launch_recurrence<T, 8, 16, 16, 2>(pp, n_items, s);
    }
    if (pp.dim <= 256) return launch_recurrence<T, 8, 32, 16, 2>(pp, n_items, s);
    return launch_recurrence<T, 32, 32, 4, 1>(pp, n_items, s);
}

extern "C" int mllm_hybrid_linear_recurrence(const RecurrenceParams* params, int n_items, int n_tokens, int dtype, void* stream) {
    if (n_items <= 0) return 0;
    const RecurrenceParams& pp = *params;
    if (pp.dim <= 0 || pp.dim > 1024 || pp.vdim <= 0) return fail("linear_recurrence: the key size must be in 1..1024");
    if (pp.qk_heads <= 0 || pp.heads % pp.qk_heads != 0) return fail("linear_recurrence: heads must be a multiple of the query/key heads");
    if (pp.heads > 65535) return fail("linear_recurrence: too many heads for one launch");
    if (pp.delta && pp.gate_b == nullptr) return fail("linear_recurrence: the delta rule needs its write gates");
    if (pp.channel_decay && pp.skip != nullptr) return fail("linear_recurrence: a decay per key channel goes with no skip");
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == DT_F32) return pick_recurrence<float>(pp, n_items, n_tokens, s);
    if (dtype == DT_BF16) return pick_recurrence<bf16>(pp, n_items, n_tokens, s);
    return fail("linear_recurrence: unknown dtype");
}

// ---------------------------------------------------------------------------
// Routed feed-forward, the plain form: every (token, chosen expert) pair by itself.
//   route        per token: z = W_router x in 32-bit, s = sigmoid(z); the `top` experts with the
//                largest s (the lower index wins a tie) with s as the weight of their INPUT; if
//                there is a shared expert, one more pair: expert `n_experts`, input weight 1,
//                output weight sigmoid(w_shared_gate . x) (or 1 for a shared expert without a gate).
//                With `softmax_of_chosen`: z (+ a bias per expert) itself ranks the experts, the
//                chosen ones' OUTPUTS are weighed by the softmax over the chosen logits only, and
//                their inputs by 1
//   expert_up    act[pair, f] = silu(W_gate[e] x') * (W_up[e] x') with x' = weight * x
//   expert_down  hidden[t] += sum over the token's pairs of out_weight * W_down[e] act[pair] (or, with `assign`,
//                hidden[t] = that sum)
// Experts are named by a table of pointers (gate, up, down) and inner sizes, so that experts of
// different sizes (the shared one) go through the same kernels; the down matrices are column
// ranges of one matrix [width, all inner sizes], so their rows lie ld_down apart.
//
// For many tokens the same sum runs as two products over ALL experts: gates and ups of every
// expert as one matrix, the down matrices side by side as another.  An expert a token did not
// choose gets the input weight 0, and expert(0) = W_down (silu(0) * 0) = 0 exactly; the input
// weight multiplies the product's result instead of its input (W (s x) = s (W x)):
//   expert_combine   act[t, c] = silu(s G[t, c]) * (s U[t, c]) * out_weight for column c of expert e,
//                    s = the token's input weight for e, or 0
// ---------------------------------------------------------------------------
// Sixteen bytes of a row as 32-bit floats in registers: 8 bfloat16 or 4 floats.
template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float* out) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        out[0] = v.x, out[1] = v.y, out[2] = v.z, out[3] = v.w;
    }
};
template <> struct Vec16<bf16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const bf16* p, float* out) {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        out[0] = __uint_as_float(v.x << 16), out[1] = __uint_as_float(v.x & 0xffff0000u);
        out[2] = __uint_as_float(v.y << 16), out[3] = __uint_as_float(v.y & 0xffff0000u);
        out[4] = __uint_as_float(v.z << 16), out[5] = __uint_as_float(v.z & 0xffff0000u);
        out[6] = __uint_as_float(v.w << 16), out[7] = __uint_as_float(v.w & 0xffff0000u);
    }
};
__device__ __forceinline__ bool aligned16(const void* p) { return (reinterpret_cast<unsigned long long>(p) & 15ull) == 0; }
static bool aligned_host(const void* p) { return (reinterpret_cast<unsigned long long>(p) & 15ull) == 0; }

template <typename T>
__global__ void __launch_bounds__(128)
route_kernel(const T* __restrict__ x, long ld_x, const T* __restrict__ router, const float* __restrict__ router_bias,
             const T* __restrict__ shared_gate, int shared_plain, int softmax_of_chosen, int width, int n_experts, int top,
             int pairs, int* __restrict__ choice, float* __restrict__ in_weight, float* __restrict__ out_weight) {
    dependents_may_start();
    wait_for_earlier_kernels();
    extern __shared__ float shared[];
    float* row = shared;                       // [width]
    float* score = row + width;                // [n_experts + 1]
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int c = threadIdx.x; c < width; c += blockDim.x) row[c] = to_f32(x[(long)t * ld_x + c]);
    __syncthreads();
    for (int e = warp; e < n_experts + (shared_gate != nullptr ? 1 : 0); e += 4) {
        const T* w = e < n_experts ? router + (long)e * width : shared_gate;
        float z = 0.0f;
        for (int c = lane; c < width; c += 32) z = fmaf(to_f32(w[c]), row[c], z);
        z = warp_sum(z);
        if (e < n_experts && router_bias != nullptr) z += router_bias[e];
        // (the chosen logits' softmax needs the logits themselves)
        if (lane == 0) score[e] = softmax_of_chosen && e < n_experts ? z : sigmoid_f(z);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float largest = 0.0f, total = 0.0f;
        for (int k = 0; k < top; k++) {
            int best = -1;
            float best_score = -INFINITY;
            for (int e = 0; e < n_experts; e++)
                if (score[e] > best_score) best = e, best_score = score[e];
            if (best < 0) best = 0, best_score = score[0];      // (scores that are no numbers)
            choice[(long)t * pairs + k] = best;
            if (softmax_of_chosen) {
                // weights of the outputs: the softmax over the chosen logits only (the first is the largest)
                if (k == 0) largest = best_score;
                const float e = expf(best_score - largest);
                in_weight[(long)t * pairs + k] = 1.0f;
                out_weight[(long)t * pairs + k] = e;
                total += e;
            } else {
                in_weight[(long)t * pairs + k] = best_score;
                out_weight[(long)t * pairs + k] = 1.0f;
            }
            score[best] = -INFINITY;
        }
        if (softmax_of_chosen)
            for (int k = 0; k < top; k++) out_weight[(long)t * pairs + k] /= total;
        if (shared_gate != nullptr || shared_plain) {
            choice[(long)t * pairs + top] = n_experts;
            in_weight[(long)t * pairs + top] = 1.0f;
            out_weight[(long)t * pairs + top] = shared_gate != nullptr ? score[n_experts] : 1.0f;
        }
    }
}

constexpr int UP_FEATURES = 32;                // inner features a block of expert_up takes (four a warp)

template <typename T>
__global__ void __launch_bounds__(256)
expert_up_kernel(T* __restrict__ act, long ld_act, const T* __restrict__ x, long ld_x, const int* __restrict__ choice,
                 const float* __restrict__ in_weight, const long long* __restrict__ gate_of, const long long* __restrict__ up_of,
                 const int* __restrict__ inner_of, int width, int pairs) {
    dependents_may_start();
    wait_for_earlier_kernels();
    extern __shared__ float row[];             // [width]: the token times its weight, rounded as an activation
    const int pair = blockIdx.x, t = pair / pairs;
    const int e = choice[pair];
    const int inner = inner_of[e];
    const int first = blockIdx.y * UP_FEATURES;
    if (first >= inner) return;
    const float weight = in_weight[pair];
    for (int c = threadIdx.x; c < width; c += blockDim.x)
        row[c] = to_f32(from_f32<T>(weight * to_f32(x[(long)t * ld_x + c])));
    __syncthreads();
    const T* gate = (const T*)gate_of[e];
    const T* up = (const T*)up_of[e];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int f = first + warp; f < min(first + UP_FEATURES, inner); f += 8) {
        const T* g = gate + (long)f * width;
        const T* u = up + (long)f * width;
        float zg = 0.0f, zu = 0.0f;
        constexpr int N = Vec16<T>::N;
        if (width % N == 0 && aligned16(g) && aligned16(u)) {
            for (int c = lane * N; c < width; c += 32 * N) {
                float a[N], b[N];
                Vec16<T>::load(g + c, a);
                Vec16<T>::load(u + c, b);
#pragma unroll
                for (int i = 0; i < N; i++) zg = fmaf(a[i], row[c + i], zg), zu = fmaf(b[i], row[c + i], zu);
            }
        } else {
            for (int c = lane; c < width; c += 32) {
                zg = fmaf(to_f32(g[c]), row[c], zg);
                zu = fmaf(to_f32(u[c]), row[c], zu);
            }
        }
        zg = warp_sum(zg), zu = warp_sum(zu);
        if (lane == 0) act[(long)pair * ld_act + f] = from_f32<T>(silu_f(zg) * zu);
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
expert_down_kernel(float* __restrict__ hidden, long ld_hidden, const T* __restrict__ act, long ld_act,
                   const int* __restrict__ choice, const float* __restrict__ out_weight, const long long* __restrict__ down_of,
                   const int* __restrict__ inner_of, long ld_down, int width, int pairs, int assign) {
    dependents_may_start();
    wait_for_earlier_kernels();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int c = blockIdx.y * 8 + warp; c < width; c += gridDim.y * 8) {
        float total = 0.0f;
        for (int k = 0; k < pairs; k++) {
            const long pair = (long)t * pairs + k;
            const int e = choice[pair];
            const int inner = inner_of[e];
            const T* w = (const T*)down_of[e] + (long)c * ld_down;
            const T* a = act + pair * ld_act;
            float z = 0.0f;
            constexpr int N = Vec16<T>::N;
            if (inner % N == 0 && aligned16(w) && aligned16(a)) {
                for (int f = lane * N; f < inner; f += 32 * N) {
                    float x[N], y[N];
                    Vec16<T>::load(w + f, x);
                    Vec16<T>::load(a + f, y);
#pragma unroll
                    for (int i = 0; i < N; i++) z = fmaf(x[i], y[i], z);
                }
            } else {
                for (int f = lane; f < inner; f += 32) z = fmaf(to_f32(w[f]), to_f32(a[f]), z);
            }
            total = fmaf(out_weight[pair], warp_sum(z), total);
        }
        if (lane == 0) hidden[(long)t * ld_hidden + c] = assign ? total : hidden[(long)t * ld_hidden + c] + total;
    }
}

// gu: [T, 2 * total] = [gates of all experts | ups of all experts]; act: [T, total].  Columns
// [e * inner, (e + 1) * inner) belong to routed expert e, columns from n_experts * inner on to the
// shared expert (pair index `top` of every token, if there is one).
// (VEC: a thread takes the 16 bytes of columns that lie side by side, all of one expert: inner sizes that are
// multiples of a vector's elements.  The token's weights per expert lie in shared memory, 0 for an expert it
// did not choose, whose columns are written as zeros without reading the products.)
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
expert_combine_kernel(T* __restrict__ act, long ld_act, const T* __restrict__ gu, long ld_gu, const int* __restrict__ choice,
                      const float* __restrict__ in_weight, const float* __restrict__ out_weight, int n_experts, int inner,
                      int total, int top, int pairs) {
    dependents_may_start();
    wait_for_earlier_kernels();
    extern __shared__ float weights[];             // [n_experts + 1][2]: input weight, output weight
    const int t = blockIdx.x;
    for (int e = threadIdx.x; e <= n_experts; e += blockDim.x) {
        float s = 0.0f, o = 1.0f;
        if (e == n_experts) {
            if (pairs > top) s = in_weight[(long)t * pairs + top], o = out_weight[(long)t * pairs + top];
        } else {
            for (int k = 0; k < top; k++)
                if (choice[(long)t * pairs + k] == e) s = in_weight[(long)t * pairs + k], o = out_weight[(long)t * pairs + k];
        }
        weights[2 * e] = s, weights[2 * e + 1] = o;
    }
    __syncthreads();
    constexpr int N = VEC ? Vec16<T>::N : 1;
    const T* row = gu + (long)t * ld_gu;
    T* dst = act + (long)t * ld_act;
    for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * N; c < total; c += gridDim.y * blockDim.x * N) {
        const int e = c < n_experts * inner ? c / inner : n_experts;
        const float s = weights[2 * e], o = weights[2 * e + 1];
        if (VEC) {
            uint4 packed = make_uint4(0u, 0u, 0u, 0u);
            if (s != 0.0f) {
                float g[N], u[N];
                Vec16<T>::load(row + c, g);
                Vec16<T>::load(row + total + c, u);
                T* lanes = reinterpret_cast<T*>(&packed);
#pragma unroll
                for (int i = 0; i < N; i++) lanes[i] = from_f32<T>(silu_f(s * g[i]) * (s * u[i]) * o);
            }
            *reinterpret_cast<uint4*>(dst + c) = packed;
        } else {
            float v = 0.0f;
            if (s != 0.0f) v = silu_f(s * to_f32(row[c])) * (s * to_f32(row[total + c])) * o;
            dst[c] = from_f32<T>(v);
        }
    }
}

extern "C" int mllm_hybrid_expert_combine(void* act, long ld_act, const void* gu, long ld_gu, const int* choice,
                                          const float* in_weight, const float* out_weight, int n_experts, int inner, int total,
                                          int top, int pairs, int n_tokens, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (dtype != DT_F32 && dtype != DT_BF16) return fail("expert_combine: unknown dtype");
    cudaStream_t s = (cudaStream_t)stream;
    const int n = dtype == DT_F32 ? 4 : 8;
    const bool vec = inner % n == 0 && total % n == 0 && ld_act % n == 0 && ld_gu % n == 0 && aligned_host(act) && aligned_host(gu);
    const int per_block = 256 * (vec ? n : 1);
    int y = (total + per_block - 1) / per_block;
    if (y > 64) y = 64;
    dim3 grid(n_tokens, y);
    const size_t shared = sizeof(float) * 2 * ((size_t)n_experts + 1);
    if (shared > 48 * 1024) return fail("expert_combine: too many experts for the table of weights");
#define RUN(T, VEC)                                                                                                             \
    launch_kernel(g_dependent_launch != 0, expert_combine_kernel<T, VEC>, grid, dim3(256), shared, s, (T*)act, ld_act, (const T*)gu, \
                  ld_gu, choice, in_weight, out_weight, n_experts, inner, total, top, pairs)
    if (dtype == DT_F32) { if (vec) RUN(float, true); else RUN(float, false); }
    else { if (vec) RUN(bf16, true); else RUN(bf16, false); }
#undef RUN
    return check_launch("expert_combine_kernel");
}

extern "C" int mllm_hybrid_route(const void* x, long ld_x, const void* router, const float* router_bias, const void* shared_gate,
                                 int shared_plain, int softmax_of_chosen, int width, int n_experts, int top, int* choice,
                                 float* in_weight, float* out_weight, int n_tokens, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (top <= 0 || top > n_experts) return fail("route: every token takes between one and all experts");
    if (shared_plain && shared_gate != nullptr) return fail("route: the shared expert has a gate or none");
    cudaStream_t s = (cudaStream_t)stream;
    const int pairs = top + (shared_gate != nullptr || shared_plain ? 1 : 0);
    const size_t shared = sizeof(float) * ((size_t)width + n_experts + 1);
    if (shared > 48 * 1024) return fail("route: the token and the scores do not fit shared memory");
    if (dtype == DT_F32)
        launch_kernel(g_dependent_launch != 0, route_kernel<float>, dim3(n_tokens), dim3(128), shared, s, (const float*)x, ld_x,
                      (const float*)router, router_bias, (const float*)shared_gate, shared_plain, softmax_of_chosen, width,
                      n_experts, top, pairs, choice, in_weight, out_weight);
    else if (dtype == DT_BF16)
        launch_kernel(g_dependent_launch != 0, route_kernel<bf16>, dim3(n_tokens), dim3(128), shared, s, (const bf16*)x, ld_x,
                      (const bf16*)router, router_bias, (const bf16*)shared_gate, shared_plain, softmax_of_chosen, width,
                      n_experts, top, pairs, choice, in_weight, out_weight);
    else
        return fail("route: unknown dtype");
    return check_launch("route_kernel");
}

extern "C" int mllm_hybrid_experts(float* hidden, long ld_hidden, void* act, long ld_act, const void* x, long ld_x,
                                   const int* choice, const float* in_weight, const float* out_weight,
                                   const long long* gate_of, const long long* up_of, const long long* down_of,
                                   const int* inner_of, long ld_down, int max_inner, int width, int pairs, int n_tokens,
                                   int assign, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t shared = sizeof(float) * (size_t)width;
    if (shared > 48 * 1024) return fail("experts: the token does not fit shared memory");
    dim3 up_grid(n_tokens * pairs, (max_inner + UP_FEATURES - 1) / UP_FEATURES);
    if (up_grid.y > 65535) return fail("experts: the inner size is too large for one launch");
    int down_y = (width + 7) / 8;
    if (down_y > 16) down_y = 16;
    dim3 down_grid(n_tokens, down_y);
    if (dtype == DT_F32) {
        launch_kernel(g_dependent_launch != 0, expert_up_kernel<float>, up_grid, dim3(256), shared, s, (float*)act, ld_act,
                      (const float*)x, ld_x, choice, in_weight, gate_of, up_of, inner_of, width, pairs);
        launch_kernel(g_dependent_launch != 0, expert_down_kernel<float>, down_grid, dim3(256), 0, s, hidden, ld_hidden,
                      (const float*)act, ld_act, choice, out_weight, down_of, inner_of, ld_down, width, pairs, assign);
    } else if (dtype == DT_BF16) {
        launch_kernel(g_dependent_launch != 0, expert_up_kernel<bf16>, up_grid, dim3(256), shared, s, (bf16*)act, ld_act,
                      (const bf16*)x, ld_x, choice, in_weight, gate_of, up_of, inner_of, width, pairs);
        launch_kernel(g_dependent_launch != 0, expert_down_kernel<bf16>, down_grid, dim3(256), 0, s, hidden, ld_hidden,
                      (const bf16*)act, ld_act, choice, out_weight, down_of, inner_of, ld_down, width, pairs, assign);
    } else {
        return fail("experts: unknown dtype");
    }
    return check_launch("expert kernels");
}

// ---------------------------------------------------------------------------
// x[r, c] += a * u[r, c] + b * v[r, c]  (32-bit; v may be null; with `assign` x is set to the sum instead)
// ---------------------------------------------------------------------------
__global__ void scaled_add_kernel(float* __restrict__ x, const float* __restrict__ u, float a, const float* __restrict__ v,
                                  float b, long n, int assign) {
    dependents_may_start();
    wait_for_earlier_kernels();
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        float sum = a * u[i];
        if (v != nullptr) sum = fmaf(b, v[i], sum);
        x[i] = assign ? sum : x[i] + sum;
    }
}

extern "C" int mllm_hybrid_scaled_add(float* x, const float* u, float a, const float* v, float b, long n, int assign, void* stream) {
    if (n <= 0) return 0;
    long blocks = (n + 255) / 256;
    if (blocks > 4096) blocks = 4096;
    launch_kernel(g_dependent_launch != 0, scaled_add_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, x, u, a, v, b, n, assign);
    return check_launch("scaled_add_kernel");
}

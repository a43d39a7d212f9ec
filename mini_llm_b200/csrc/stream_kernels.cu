// Kernels of layers whose residual is several streams (hyper-connections), and of gated feed-forwards:
//   streams_fill   every stream of a token starts as the token's embedded row
//   streams_step   per token, one block: (1) if a sublayer result y is given, all streams at once from
//                  the old ones, x_t <- sum_s mix[s, t] x_s + out[t] y; (2) if asked, the read-out
//                  u = sum_s in[s] x_s of the (new) streams (in = null: the plain sum), stored in
//                  32-bit and / or divided by its root mean square and multiplied by a gain, as the
//                  input of the next sublayer.  Streams, weights and sums are 32-bit.
//   gated_act      act(gate) * up over the two halves of a product's result
// The normed read-out is templated on the element type of the activations (float: the true 32-bit
// path; bfloat16: the serving path); every kernel is launched as a programmatic dependent of the
// kernel before it.
#include "common.cuh"

MLLM_DEFINE_ERROR_API(mllm_streams)

constexpr int MAX_STREAMS = 16;

__global__ void streams_fill_kernel(float* __restrict__ streams, const float* __restrict__ hidden, int n_streams, int width,
                                    long n) {
    dependents_may_start();
    wait_for_earlier_kernels();
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;         // over tokens * width
    if (i >= n) return;
    const long t = i / width, c = i % width;
    const float v = hidden[i];
    for (int s = 0; s < n_streams; s++) streams[(t * n_streams + s) * width + c] = v;
}

extern "C" int mllm_streams_fill(float* streams, const float* hidden, int n_streams, int width, int n_tokens, void* stream) {
    if (n_tokens <= 0) return 0;
    if (n_streams <= 0 || width <= 0) return fail("streams_fill: sizes must be positive");
    const long n = (long)n_tokens * width;
    launch_kernel(g_dependent_launch != 0, streams_fill_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, (cudaStream_t)stream,
                  streams, hidden, n_streams, width, n);
    return check_launch("streams_fill_kernel");
}

// VEC: 4 (every row starts on a 16-byte boundary and the width is a multiple of four: four columns a thread,
// moved as one vector) or 1.  NS: the number of streams where it is known when compiled (1 to 4: the sums
// unroll to what is needed and the kernel's registers allow more blocks an SM), 0 for any number up to 8, -1 for
// any number up to 16.
template <typename T, int VEC, int NS>
__global__ void __launch_bounds__(256)
streams_step_kernel(float* __restrict__ streams, const float* __restrict__ y, long ld_y, const float* __restrict__ mix,
                    const float* __restrict__ w_out, int read, const float* __restrict__ w_in, float* __restrict__ u_out,
                    long ld_u, T* __restrict__ normed, long ld_normed, const float* __restrict__ gain, float eps, int n_streams,
                    int width) {
    constexpr int BOUND = NS > 0 ? NS : (NS == 0 ? 8 : MAX_STREAMS);
    if (NS > 0) n_streams = NS;
    dependents_may_start();
    wait_for_earlier_kernels();
    extern __shared__ float u_row[];                 // [width]: the read-out, until it is normed
    __shared__ float scratch[33];
    __shared__ float m[MAX_STREAMS * MAX_STREAMS], o[MAX_STREAMS], in[MAX_STREAMS];
    const int t = blockIdx.x;
    if (threadIdx.x < n_streams * n_streams && y != nullptr) m[threadIdx.x] = mix[threadIdx.x];
    if (threadIdx.x < n_streams) {
        if (y != nullptr) o[threadIdx.x] = w_out[threadIdx.x];
        in[threadIdx.x] = w_in != nullptr ? w_in[threadIdx.x] : 1.0f;
    }
    __syncthreads();
    float* mine = streams + (long)t * n_streams * width;
    float sq = 0.0f;
    for (int c = threadIdx.x * VEC; c < width; c += blockDim.x * VEC) {
        alignas(16) float x[BOUND][VEC];
#pragma unroll
        for (int s = 0; s < BOUND; s++) {
            if (s < n_streams) {
                if constexpr (VEC == 4)
                    *reinterpret_cast<float4*>(x[s]) = *reinterpret_cast<const float4*>(mine + (long)s * width + c);
                else
                    x[s][0] = mine[(long)s * width + c];
            } else {
#pragma unroll
                for (int e = 0; e < VEC; e++) x[s][e] = 0.0f;
            }
        }
        // the read-out of the streams as they then are; a new stream goes to memory as soon as it is summed (the old
        // ones stay in registers until all are), and into the read-out
        alignas(16) float u[VEC];
#pragma unroll
        for (int e = 0; e < VEC; e++) u[e] = 0.0f;
        if (y != nullptr) {
            alignas(16) float result[VEC];
            if constexpr (VEC == 4)
                *reinterpret_cast<float4*>(result) = *reinterpret_cast<const float4*>(y + (long)t * ld_y + c);
            else
                result[0] = y[(long)t * ld_y + c];
#pragma unroll
            for (int to = 0; to < BOUND; to++) {
                if (to >= n_streams) continue;
                alignas(16) float fresh[VEC];
#pragma unroll
                for (int e = 0; e < VEC; e++) {
                    float sum = 0.0f;
#pragma unroll
                    for (int s = 0; s < BOUND; s++)
                        if (s < n_streams) sum = fmaf(m[s * n_streams + to], x[s][e], sum);
                    fresh[e] = fmaf(o[to], result[e], sum);
                    u[e] = fmaf(in[to], fresh[e], u[e]);
                }
                if constexpr (VEC == 4)
                    *reinterpret_cast<float4*>(mine + (long)to * width + c) = *reinterpret_cast<const float4*>(fresh);
                else
                    mine[(long)to * width + c] = fresh[0];
            }
        } else {
#pragma unroll
            for (int s = 0; s < BOUND; s++)
                if (s < n_streams) {
#pragma unroll
                    for (int e = 0; e < VEC; e++) u[e] = fmaf(in[s], x[s][e], u[e]);
                }
        }
        if (read) {
#pragma unroll
            for (int e = 0; e < VEC; e++) {
                if (u_out != nullptr) u_out[(long)t * ld_u + c + e] = u[e];
                u_row[c + e] = u[e];
                sq = fmaf(u[e], u[e], sq);
            }
        }
    }
    if (!read || normed == nullptr) return;
    // (every thread reads back the columns it wrote itself: no barrier is needed before the sum's own)
    const float inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)width + eps);
    for (int c = threadIdx.x * VEC; c < width; c += blockDim.x * VEC) {
#pragma unroll
        for (int e = 0; e < VEC; e++) normed[(long)t * ld_normed + c + e] = from_f32<T>(u_row[c + e] * inv * gain[c + e]);
    }
}

extern "C" int mllm_streams_step(float* streams, const float* y, long ld_y, const float* mix, const float* w_out, int read,
                                 const float* w_in, float* u_out, long ld_u, void* normed, long ld_normed, const float* gain,
                                 float eps, int n_streams, int width, int n_tokens, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (n_streams <= 0 || n_streams > MAX_STREAMS) return fail("streams_step: between 1 and 16 streams");
    if (width <= 0) return fail("streams_step: the width must be positive");
    if (y != nullptr && (mix == nullptr || w_out == nullptr)) return fail("streams_step: a sublayer result needs its mixing weights");
    if (normed != nullptr && (gain == nullptr || !read)) return fail("streams_step: the normed read-out needs a gain");
    const size_t shared = (size_t)width * sizeof(float);
    if (shared > 200 * 1024) return fail("streams_step: the row does not fit in shared memory");
    cudaStream_t s = (cudaStream_t)stream;
    // (more than 8 streams: a column a thread, so that a thread's old streams stay in registers)
    const bool vec = n_streams <= 8 && width % 4 == 0 && ((uintptr_t)streams & 15) == 0 &&
                     (y == nullptr || (((uintptr_t)y & 15) == 0 && ld_y % 4 == 0));
#define LAUNCH_STREAMS_AS(T, VEC, NS)                                                                                            \
    do {                                                                                                                         \
        if (shared > 48 * 1024)                                                                                                  \
            cudaFuncSetAttribute(streams_step_kernel<T, VEC, NS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);     \
        launch_kernel(g_dependent_launch != 0, streams_step_kernel<T, VEC, NS>, dim3(n_tokens), dim3(256), shared, s, streams,   \
                      y, ld_y, mix, w_out, read, w_in, u_out, ld_u, (T*)normed, ld_normed, gain, eps, n_streams, width);         \
    } while (0)
#define LAUNCH_STREAMS(T, VEC)                                                                                                   \
    do {                                                                                                                         \
        switch (n_streams) {                                                                                                     \
        case 1: LAUNCH_STREAMS_AS(T, VEC, 1); break;                                                                             \
        case 2: LAUNCH_STREAMS_AS(T, VEC, 2); break;                                                                             \
        case 3: LAUNCH_STREAMS_AS(T, VEC, 3); break;                                                                             \
        case 4: LAUNCH_STREAMS_AS(T, VEC, 4); break;                                                                             \
        default:                                                                                                                 \
            if (n_streams <= 8) LAUNCH_STREAMS_AS(T, VEC, 0); else LAUNCH_STREAMS_AS(T, 1, -1);                                  \
            break;                                                                                                               \
        }                                                                                                                        \
    } while (0)
    if (dtype == DT_F32) {
        if (vec) LAUNCH_STREAMS(float, 4); else LAUNCH_STREAMS(float, 1);
    } else if (dtype == DT_BF16) {
        if (vec) LAUNCH_STREAMS(bf16, 4); else LAUNCH_STREAMS(bf16, 1);
    } else {
        return fail("streams_step: unknown dtype");
    }
#undef LAUNCH_STREAMS_AS
#undef LAUNCH_STREAMS
    return check_launch("streams_step_kernel");
}

// out[t, f] = act(gu[t, f]) * gu[t, inner + f]; act: 0 silu, 1 gelu (tanh form), 2 none.  VEC entries a thread:
// 16 bytes where every row and both halves start on such a boundary, else one.
template <typename T, int VEC>
__global__ void gated_act_kernel(T* __restrict__ out, long ld_out, const T* __restrict__ gu, long ld_gu, int inner, int act,
                                 long n) {
    dependents_may_start();
    wait_for_earlier_kernels();
    const long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    if (i >= n) return;
    const long t = i / inner, f = i % inner;
    struct alignas(sizeof(T) * VEC) Pack { T e[VEC]; };
    const Pack gate = *reinterpret_cast<const Pack*>(gu + t * ld_gu + f);
    const Pack up = *reinterpret_cast<const Pack*>(gu + t * ld_gu + inner + f);
    Pack result;
#pragma unroll
    for (int e = 0; e < VEC; e++) {
        const float g = to_f32(gate.e[e]);
        const float a = act == 0 ? g / (1.0f + expf(-g)) : (act == 1 ? gelu_tanh_f(g) : g);
        result.e[e] = from_f32<T>(a * to_f32(up.e[e]));
    }
    *reinterpret_cast<Pack*>(out + t * ld_out + f) = result;
}

extern "C" int mllm_streams_gated_act(void* out, long ld_out, const void* gu, long ld_gu, int inner, int act, int n_tokens,
                                      int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (inner <= 0 || act < 0 || act > 2) return fail("gated_act: bad sizes or activation");
    const long n = (long)n_tokens * inner;
    cudaStream_t s = (cudaStream_t)stream;
    const int size = dtype == DT_F32 ? 4 : 2, wide = 16 / size;
    const bool vec = inner % wide == 0 && ld_gu % wide == 0 && ld_out % wide == 0 && ((uintptr_t)gu & 15) == 0 && ((uintptr_t)out & 15) == 0;
#define LAUNCH_GATED(T, VEC)                                                                                                   \
    launch_kernel(g_dependent_launch != 0, gated_act_kernel<T, VEC>, dim3((unsigned)((n / VEC + 255) / 256)), dim3(256), 0, s, \
                  (T*)out, ld_out, (const T*)gu, ld_gu, inner, act, n)
    if (dtype == DT_F32) {
        if (vec) LAUNCH_GATED(float, 4); else LAUNCH_GATED(float, 1);
    } else if (dtype == DT_BF16) {
        if (vec) LAUNCH_GATED(bf16, 8); else LAUNCH_GATED(bf16, 1);
    } else {
        return fail("gated_act: unknown dtype");
    }
#undef LAUNCH_GATED
    return check_launch("gated_act_kernel");
}

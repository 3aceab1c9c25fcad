// A residual stream held as several copies (hyper-connections), and the embedding that opens it.
//
// A token's row holds S streams of `hidden` floats, one after another.  Around a sublayer with
// coefficients in[S], out[S] and mix[S, S] (first index: the copy read; second: the copy written) the streams move as
//     u   = sum_s in[s] x_s                      what the sublayer's norm reads
//     y   = sublayer(norm(u))
//     x_t = sum_s mix[s, t] x_s + out[t] y       all t at once, from the old streams
// ns_stream_mix_norm does, for one row and in one pass, the second half of the sublayer before (its y is
// still pending: the streams are rewritten in place) and the first half of the next one (u and its norm).
// With in == null every stream counts once (the sum that closes the model); with mix == null and
// out == null the step is x += y.  One stream, no coefficients: the residual sum and a norm, which is
// how a layer norm with a bias runs on a plain stream.  The norm is an RMS norm or, `centered`, a layer
// norm (mean of the squared deviations), with an optional bias; statistics, gain and bias are float and
// the result is rounded once.
#include "common.cuh"

namespace {

constexpr int kMaxStreams = 16;  // the kernels are built for up to 4, 8 and 16 copies

__device__ __forceinline__ void ld4(const float* p, float (&v)[4]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
}
__device__ __forceinline__ void ld4(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}

template <typename T, int VEC, int MAXS>
__global__ void __launch_bounds__(256)
stream_mix_norm_kernel(float* __restrict__ streams, const T* __restrict__ y, const float* __restrict__ mix,
                       const float* __restrict__ outw, const float* __restrict__ inw, const float* __restrict__ gain,
                       const float* __restrict__ bias, T* __restrict__ out, const int* __restrict__ rows, int S, int hidden,
                       float eps, int centered, int write_back) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    extern __shared__ float u_row[];
    __shared__ float scratch[32];
    __shared__ float c_mix[MAXS * MAXS], c_out[MAXS], c_in[MAXS];
    const int j = blockIdx.x, tid = threadIdx.x;
    const int row = rows ? rows[j] : j;
    for (int i = tid; i < S * S; i += blockDim.x) c_mix[i] = mix ? mix[i] : (i / S == i % S ? 1.f : 0.f);
    if (tid < S) {
        c_out[tid] = outw ? outw[tid] : 1.f;
        c_in[tid] = inw ? inw[tid] : 1.f;
    }
    __syncthreads();
    float* xs = streams + (size_t)row * S * hidden;
    const T* yr = y ? y + (size_t)row * hidden : nullptr;
    float sum = 0.f;
    // four neighbouring features per thread and turn when rows start on 16 bytes (VEC), one otherwise
    for (int h = tid * VEC; h < hidden; h += blockDim.x * VEC) {
        float x[MAXS][VEC];
#pragma unroll
        for (int s = 0; s < MAXS; ++s) {
            if (s < S) {
                if constexpr (VEC == 4) {
                    const float4 v = *reinterpret_cast<const float4*>(xs + (size_t)s * hidden + h);
                    x[s][0] = v.x; x[s][1] = v.y; x[s][2] = v.z; x[s][3] = v.w;
                } else {
                    x[s][0] = xs[(size_t)s * hidden + h];
                }
            } else {
#pragma unroll
                for (int i = 0; i < VEC; ++i) x[s][i] = 0.f;
            }
        }
        if (yr) {
            float yv[VEC];
            if constexpr (VEC == 4) ld4(yr + h, yv); else yv[0] = ns_ld(yr, h);
            float nx[MAXS][VEC];
#pragma unroll
            for (int t = 0; t < MAXS; ++t) {
#pragma unroll
                for (int i = 0; i < VEC; ++i) {
                    float a = 0.f;
                    if (t < S) {
#pragma unroll
                        for (int s = 0; s < MAXS; ++s)
                            if (s < S) a = fmaf(c_mix[s * S + t], x[s][i], a);
                        a = fmaf(c_out[t], yv[i], a);
                    }
                    nx[t][i] = a;
                }
            }
#pragma unroll
            for (int t = 0; t < MAXS; ++t) {
#pragma unroll
                for (int i = 0; i < VEC; ++i) x[t][i] = nx[t][i];
                if (write_back && t < S) {
                    if constexpr (VEC == 4) *reinterpret_cast<float4*>(xs + (size_t)t * hidden + h) = make_float4(nx[t][0], nx[t][1], nx[t][2], nx[t][3]);
                    else xs[(size_t)t * hidden + h] = nx[t][0];
                }
            }
        }
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            float u = 0.f;
#pragma unroll
            for (int s = 0; s < MAXS; ++s)
                if (s < S) u = fmaf(c_in[s], x[s][i], u);
            u_row[h + i] = u;
            sum += centered ? u : u * u;
        }
    }
    if (!out) return;  // only the streams were wanted
    T* o = out + (size_t)j * hidden;
    float mean = 0.f, inv;
    if (centered) {
        mean = ns_block_sum(sum, scratch) / (float)hidden;
        float ss = 0.f;
        for (int h = tid; h < hidden; h += blockDim.x) {
            const float d = u_row[h] - mean;
            ss += d * d;
        }
        inv = 1.f / sqrtf(ns_block_sum(ss, scratch) / (float)hidden + eps);
    } else {
        inv = 1.f / sqrtf(ns_block_sum(sum, scratch) / (float)hidden + eps);
    }
    for (int h = tid; h < hidden; h += blockDim.x) {
        float v = (u_row[h] - mean) * inv * gain[h];
        if (bias) v += bias[h];
        ns_st(o, h, v);
    }
}

// sum_out[j, :] = sum_s in[s] x_s of row rows[j] (after a pending write that is applied on the fly and not stored)
template <typename T>
__global__ void __launch_bounds__(256)
stream_read_kernel(const float* __restrict__ streams, const T* __restrict__ y, const float* __restrict__ mix,
                   const float* __restrict__ outw, const float* __restrict__ inw, float* __restrict__ sum_out, int S,
                   int hidden, size_t total) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t row = i / hidden;
    const int h = (int)(i - row * hidden);
    const float* xs = streams + row * S * hidden;
    const float yv = y ? ns_ld(y, i) : 0.f;
    float u = 0.f;
    for (int t = 0; t < S; ++t) {
        float a;
        if (y) {
            a = 0.f;
            for (int s = 0; s < S; ++s) a = fmaf(mix ? mix[s * S + t] : (s == t ? 1.f : 0.f), xs[(size_t)s * hidden + h], a);
            a = fmaf(outw ? outw[t] : 1.f, yv, a);
        } else {
            a = xs[(size_t)t * hidden + h];
        }
        u = fmaf(inw ? inw[t] : 1.f, a, u);
    }
    sum_out[i] = u;
}

template <typename T>
__global__ void embed_streams_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                                     int hidden, int vocab, float scale, int copies) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    const int n = blockIdx.x;
    const int id = ids[n];
    float* o = out + (size_t)n * copies * hidden;
    const bool ok = id >= 0 && id < vocab;
    const T* row = table + (size_t)(ok ? id : 0) * hidden;
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
        const float v = ok ? ns_ld(row, h) * scale : 0.f;
        for (int s = 0; s < copies; ++s) o[(size_t)s * hidden + h] = v;
    }
}

}  // namespace

// streams [rows, S * hidden] float, rewritten in place when y is given and no row selection is;
// y [rows, hidden] or null; mix [S, S], outw [S], inw [S] float or null (see above); out [n_rows, hidden]
// or null; rows: output row j reads row rows[j] (then nothing is written back).
NS_API int ns_stream_mix_norm(float* streams, const void* y, const float* mix, const float* outw, const float* inw,
                              const float* gain, const float* bias, void* out, const int* rows, int n_rows, int S,
                              int hidden, float eps, int centered, int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return NS_OK;
    if (S < 1 || S > kMaxStreams) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_stream_mix_norm: %d streams (1 to %d are built)", S, kMaxStreams);
    if (hidden <= 0) NS_FAIL(NS_ERR_ARGUMENT, "ns_stream_mix_norm: hidden=%d", hidden);
    if (out && !gain) NS_FAIL(NS_ERR_ARGUMENT, "ns_stream_mix_norm: a norm needs its gain");
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 200 * 1024) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_stream_mix_norm: a row of %d floats does not fit shared memory", hidden);
    const int write_back = rows ? 0 : 1;
    // which kernel runs depends on the width and the alignment only, never on the batch
    const bool vec = hidden % 4 == 0 && (((uintptr_t)streams | (uintptr_t)y) % 16 == 0);
    const int threads = hidden >= 1024 ? 256 : 128;
#define NS_STREAM_LAUNCH_S(T, V, M)                                                                                              \
    {                                                                                                                            \
        if (smem > 48 * 1024) NS_CUDA(cudaFuncSetAttribute(stream_mix_norm_kernel<T, V, M>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)); \
        NS_LAUNCH((stream_mix_norm_kernel<T, V, M>), n_rows, threads, smem, stream, streams, (const T*)y, mix, outw, inw, gain, bias, (T*)out, \
                  rows, S, hidden, eps, centered, write_back);                                                                   \
    }
#define NS_STREAM_LAUNCH(T, V)                                                                                                   \
    {                                                                                                                            \
        if (S <= 4) NS_STREAM_LAUNCH_S(T, V, 4) else if (S <= 8) NS_STREAM_LAUNCH_S(T, V, 8) else NS_STREAM_LAUNCH_S(T, 1, 16)               \
    }
    if (dtype == NS_F32) {
        if (vec) NS_STREAM_LAUNCH(float, 4) else NS_STREAM_LAUNCH(float, 1)
    } else if (dtype == NS_BF16) {
        if (vec) NS_STREAM_LAUNCH(__nv_bfloat16, 4) else NS_STREAM_LAUNCH(__nv_bfloat16, 1)
    } else {
        NS_FAIL(NS_ERR_ARGUMENT, "ns_stream_mix_norm: unknown dtype %d", dtype);
    }
#undef NS_STREAM_LAUNCH
#undef NS_STREAM_LAUNCH_S
    NS_CHECK_LAUNCH("ns_stream_mix_norm");
    return NS_OK;
}

// sum_out [n_rows, hidden] float = what a sublayer with `inw` would read, every row, nothing rewritten
NS_API int ns_stream_read(const float* streams, const void* y, const float* mix, const float* outw, const float* inw,
                          float* sum_out, int n_rows, int S, int hidden, int dtype, cudaStream_t stream) {
    const size_t total = (size_t)n_rows * hidden;
    if (total == 0) return NS_OK;
    if (S < 1 || S > kMaxStreams) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_stream_read: %d streams (1 to %d are built)", S, kMaxStreams);
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == NS_F32)
        NS_LAUNCH((stream_read_kernel<float>), blocks, 256, 0, stream, streams, (const float*)y, mix, outw, inw, sum_out, S, hidden, total);
    else if (dtype == NS_BF16)
        NS_LAUNCH((stream_read_kernel<__nv_bfloat16>), blocks, 256, 0, stream, streams, (const __nv_bfloat16*)y, mix, outw, inw,
                  sum_out, S, hidden, total);
    else
        NS_FAIL(NS_ERR_ARGUMENT, "ns_stream_read: unknown dtype %d", dtype);
    NS_CHECK_LAUNCH("ns_stream_read");
    return NS_OK;
}

// out[n, s * hidden + h] = float(table[ids[n], h]) * scale for every copy s; an id outside the table gives zeros
NS_API int ns_embed_streams(const void* table, const int* ids, float* out, int n_tokens, int hidden, int vocab, float scale,
                            int copies, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return NS_OK;
    if (copies < 1) NS_FAIL(NS_ERR_ARGUMENT, "ns_embed_streams: copies=%d", copies);
    const int threads = hidden >= 1024 ? 256 : (hidden >= 256 ? 128 : 64);
    if (dtype == NS_F32)
        NS_LAUNCH((embed_streams_kernel<float>), n_tokens, threads, 0, stream, (const float*)table, ids, out, hidden, vocab, scale, copies);
    else if (dtype == NS_BF16)
        NS_LAUNCH((embed_streams_kernel<__nv_bfloat16>), n_tokens, threads, 0, stream, (const __nv_bfloat16*)table, ids, out, hidden,
                  vocab, scale, copies);
    else
        NS_FAIL(NS_ERR_ARGUMENT, "ns_embed_streams: unknown dtype %d", dtype);
    NS_CHECK_LAUNCH("ns_embed_streams");
    return NS_OK;
}

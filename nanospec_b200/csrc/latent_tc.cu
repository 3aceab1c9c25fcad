// Attention over a cached latent on the tensor cores (bfloat16, m16n8k16), for prompts and for decoding alike.
//
// The same computation as ns_attention_latent (csrc/latent.cu): one shared key head of D = R + r features whose
// first R features are also the value.  A block takes one token and up to 16 of its heads as the 16 rows of the
// tensor-core tile - the heads share every key, so a key tile is loaded once for all of them - and walks the token's
// visible keys 64 at a time:
//   S = Q K^T     each of the eight warps takes 8 of the tile's keys over all D features
//   softmax       float, running maximum and sum per row; the row statistics of the eight warps meet in shared memory
//   O += P V      each warp takes an eighth of the R value columns over all 64 keys; P goes through shared memory as
//                 a pair of bfloat16 (the rounded weight and what the rounding dropped, about 16 bits together)
// When a step has few (token, head group) pairs the keys of a token are split over several blocks, which leave
// unnormalised partial results in scratch; ns_latent_merge adds them up.  The sink joins the denominator and the
// gate's sigmoid scales the row at the very end (in the block itself when the keys are not split).
// Sizes: R and r multiples of 16, R at most 512; others are the exact kernel's.
#include "mma_utils.cuh"

namespace {

constexpr int kKeysTile = 64;
constexpr int kRows = 16;
constexpr int kWarps = 8;
constexpr int kPStride = kKeysTile + 8;
constexpr float kLog2e = 1.4426950408889634f;

// UNITS: 16-column units of the value that one warp owns (R / 128, rounded up)
template <int UNITS>
__global__ void __launch_bounds__(kWarps * 32)
attention_latent_tc_kernel(const __nv_bfloat16* __restrict__ q_lat, long long ql_tok, long long ql_head,
                           const __nv_bfloat16* __restrict__ q_rot, long long qr_tok, long long qr_head,
                           const __nv_bfloat16* __restrict__ cache, const int* __restrict__ block_table, int table_stride,
                           const int* __restrict__ token_req, const int* __restrict__ positions,
                           const float* __restrict__ sink, const __nv_bfloat16* __restrict__ gate, long long gate_tok,
                           __nv_bfloat16* __restrict__ out, long long o_tok, long long o_head, float* __restrict__ part_o,
                           float* __restrict__ part_ml, int H, int R, int r, int page_size, float scale, int window,
                           int n_splits) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int D = R + r, KS = D + 8;  // row stride of the key and query tiles in elements
    __nv_bfloat16* ks = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [64][KS]
    __nv_bfloat16* qs = ks + kKeysTile * KS;                          // [16][KS]
    __nv_bfloat16* ph = qs + kRows * KS;                              // [16][72] rounded weights
    __nv_bfloat16* pl = ph + kRows * kPStride;                        // [16][72] what the rounding dropped
    float* wmax = reinterpret_cast<float*>(pl + kRows * kPStride);    // [warps][16]
    float* wsum = wmax + kWarps * kRows;                              // [warps][16]
    __shared__ unsigned slots[kKeysTile];

    const int n = blockIdx.x, h0 = blockIdx.y * kRows, split = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int req = token_req[n];
    if (req < 0) return;
    const int pos = positions[n];
    const int kend_all = pos + 1;
    const int kstart_all = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    // this block's share of the keys: whole tiles, the same for every head group of the token
    const int tiles_all = (kend_all - kstart_all + kKeysTile - 1) / kKeysTile;
    const int tiles_per = (tiles_all + n_splits - 1) / n_splits;
    const int kstart = kstart_all + split * tiles_per * kKeysTile;
    const int kend = min(kend_all, kstart + tiles_per * kKeysTile);
    const int* bt = block_table + (size_t)req * table_stride;
    const int chunks = D / 8;  // 16-byte pieces of a row

    // the queries: rows of [q_lat | q_rot]; rows past the last head are zero
    for (int c = tid; c < kRows * chunks; c += blockDim.x) {
        const int row = c / chunks, ch = c - row * chunks;
        const int h = h0 + row;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (h < H) {
            const int e = ch * 8;
            const __nv_bfloat16* src = e < R ? q_lat + (size_t)n * ql_tok + (size_t)h * ql_head + e
                                             : q_rot + (size_t)n * qr_tok + (size_t)h * qr_head + (e - R);
            if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
                v = *reinterpret_cast<const uint4*>(src);
            } else {
                __align__(16) __nv_bfloat16 t[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) t[i] = src[i];
                v = *reinterpret_cast<const uint4*>(t);
            }
        }
        *reinterpret_cast<uint4*>(qs + row * KS + ch * 8) = v;
    }

    const float scale2 = scale * kLog2e;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;  // rows lane / 4 and lane / 4 + 8
    float o[UNITS][2][4];
#pragma unroll
    for (int u = 0; u < UNITS; ++u)
#pragma unroll
        for (int t = 0; t < 2; ++t)
#pragma unroll
            for (int i = 0; i < 4; ++i) o[u][t][i] = 0.f;
    const int n_units = R / 16;

    for (int k0 = kstart; k0 < kend; k0 += kKeysTile) {
        __syncthreads();  // the tile of the round before has been read (and, the first time, nothing)
        if (tid < kKeysTile) {
            const int key = k0 + tid;
            slots[tid] = key < kend ? (unsigned)bt[key / page_size] * (unsigned)page_size + (unsigned)(key % page_size) : 0xffffffffu;
        }
        __syncthreads();
        // a warp copies whole rows, its lanes the 16-byte pieces of a row: no division per piece
        for (int row = warp; row < kKeysTile; row += kWarps) {
            const unsigned s = slots[row];
            const __nv_bfloat16* src = cache + (s == 0xffffffffu ? 0 : (size_t)s * D);
            for (int ch = lane; ch < chunks; ch += 32) ns_cp_async16(ks + row * KS + ch * 8, src + ch * 8, s != 0xffffffffu);
        }
        ns_cp_async_commit();
        ns_cp_async_wait<0>();
        __syncthreads();

        // ---- S = Q K^T for this warp's 8 keys
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        const int kw = warp * 8;
        for (int d0 = 0; d0 < D; d0 += 16) {
            uint32_t a[4], b[2];
            ns_ldmatrix_x4(a, qs + ((lane & 7) + ((lane >> 3) & 1) * 8) * KS + d0 + (lane >> 4) * 8);
            ns_ldmatrix_x2(b, ks + (kw + (lane & 7)) * KS + d0 + ((lane >> 3) & 1) * 8);
            ns_mma_bf16(s, a, b[0], b[1]);
        }
        // scale, mask the keys past the end, this warp's row maxima
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int key = k0 + kw + (lane & 3) * 2 + (i & 1);
            s[i] = key < kend ? s[i] * scale2 : -INFINITY;
            if (i < 2) mx0 = fmaxf(mx0, s[i]); else mx1 = fmaxf(mx1, s[i]);
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        if ((lane & 3) == 0) {
            wmax[warp * kRows + (lane >> 2)] = mx0;
            wmax[warp * kRows + (lane >> 2) + 8] = mx1;
        }
        __syncthreads();
        const int r0 = lane >> 2, r1 = r0 + 8;
        float mn0 = m0, mn1 = m1;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            mn0 = fmaxf(mn0, wmax[w * kRows + r0]);
            mn1 = fmaxf(mn1, wmax[w * kRows + r1]);
        }
        const float c0 = ns_exp2(m0 - mn0), c1 = ns_exp2(m1 - mn1);  // the first tile: 2^(-inf) = 0
        m0 = mn0;
        m1 = mn1;
        const float p0 = ns_exp2(s[0] - mn0), p1 = ns_exp2(s[1] - mn0);
        const float p2 = ns_exp2(s[2] - mn1), p3 = ns_exp2(s[3] - mn1);
        float sum0 = p0 + p1, sum1 = p2 + p3;
        {
            const int col = kw + (lane & 3) * 2;
            *reinterpret_cast<uint32_t*>(ph + r0 * kPStride + col) = ns_pack_bf16(p0, p1);
            *reinterpret_cast<uint32_t*>(ph + r1 * kPStride + col) = ns_pack_bf16(p2, p3);
            *reinterpret_cast<uint32_t*>(pl + r0 * kPStride + col) = ns_pack_bf16_rest(p0, p1);
            *reinterpret_cast<uint32_t*>(pl + r1 * kPStride + col) = ns_pack_bf16_rest(p2, p3);
        }
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
        sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
        sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
        if ((lane & 3) == 0) {
            wsum[warp * kRows + r0] = sum0;
            wsum[warp * kRows + r1] = sum1;
        }
        __syncthreads();
        {
            float t0 = 0.f, t1 = 0.f;  // the warps' sums in their order
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                t0 += wsum[w * kRows + r0];
                t1 += wsum[w * kRows + r1];
            }
            l0 = l0 * c0 + t0;
            l1 = l1 * c1 + t1;
        }

        // ---- O += P V over this warp's value columns (units warp, warp + 8, ...)
#pragma unroll
        for (int u = 0; u < UNITS; ++u)
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                o[u][t][0] *= c0; o[u][t][1] *= c0;
                o[u][t][2] *= c1; o[u][t][3] *= c1;
            }
#pragma unroll
        for (int kk = 0; kk < kKeysTile / 16; ++kk) {
            uint32_t ah[4], al[4];
            const int prow = (lane & 7) + ((lane >> 3) & 1) * 8, pcol = kk * 16 + (lane >> 4) * 8;
            ns_ldmatrix_x4(ah, ph + prow * kPStride + pcol);
            ns_ldmatrix_x4(al, pl + prow * kPStride + pcol);
#pragma unroll
            for (int u = 0; u < UNITS; ++u) {
                const int unit = warp + kWarps * u;
                if (unit < n_units) {
                    uint32_t b[4];
                    ns_ldmatrix_x4_trans(b, ks + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * KS + unit * 16 + (lane >> 4) * 8);
                    ns_mma_bf16(o[u][0], ah, b[0], b[1]);
                    ns_mma_bf16(o[u][1], ah, b[2], b[3]);
                    ns_mma_bf16(o[u][0], al, b[0], b[1]);
                    ns_mma_bf16(o[u][1], al, b[2], b[3]);
                }
            }
        }
    }

    const int r0 = lane >> 2, r1 = r0 + 8;
    const int ha = h0 + r0, hb = h0 + r1;
    if (n_splits > 1) {  // unnormalised, for the merge
        const size_t item = ((size_t)n * gridDim.y + blockIdx.y) * n_splits + split;
        float* po = part_o + item * kRows * R;
        if (warp == 0 && (lane & 3) == 0) {
            part_ml[(item * kRows + r0) * 2] = m0;
            part_ml[(item * kRows + r0) * 2 + 1] = l0;
            part_ml[(item * kRows + r1) * 2] = m1;
            part_ml[(item * kRows + r1) * 2 + 1] = l1;
        }
#pragma unroll
        for (int u = 0; u < UNITS; ++u) {
            const int unit = warp + kWarps * u;
            if (unit >= n_units) continue;
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                const int col = unit * 16 + t * 8 + (lane & 3) * 2;
                *reinterpret_cast<float2*>(po + (size_t)r0 * R + col) = make_float2(o[u][t][0], o[u][t][1]);
                *reinterpret_cast<float2*>(po + (size_t)r1 * R + col) = make_float2(o[u][t][2], o[u][t][3]);
            }
        }
        return;
    }
    float f0 = 1.f, f1 = 1.f;
    if (sink) {
        if (ha < H) {
            const float sk = sink[ha] * kLog2e, mf = fmaxf(m0, sk);
            f0 = ns_exp2(m0 - mf);
            l0 = l0 * f0 + ns_exp2(sk - mf);
        }
        if (hb < H) {
            const float sk = sink[hb] * kLog2e, mf = fmaxf(m1, sk);
            f1 = ns_exp2(m1 - mf);
            l1 = l1 * f1 + ns_exp2(sk - mf);
        }
    }
    f0 /= l0;
    f1 /= l1;
    if (gate) {
        if (ha < H) f0 *= 1.f / (1.f + expf(-__bfloat162float(gate[(size_t)n * gate_tok + ha])));
        if (hb < H) f1 *= 1.f / (1.f + expf(-__bfloat162float(gate[(size_t)n * gate_tok + hb])));
    }
#pragma unroll
    for (int u = 0; u < UNITS; ++u) {
        const int unit = warp + kWarps * u;
        if (unit >= n_units) continue;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            const int col = unit * 16 + t * 8 + (lane & 3) * 2;
            if (ha < H)
                *reinterpret_cast<uint32_t*>(out + (size_t)n * o_tok + (size_t)ha * o_head + col) = ns_pack_bf16(o[u][t][0] * f0, o[u][t][1] * f0);
            if (hb < H)
                *reinterpret_cast<uint32_t*>(out + (size_t)n * o_tok + (size_t)hb * o_head + col) = ns_pack_bf16(o[u][t][2] * f1, o[u][t][3] * f1);
        }
    }
}

// one block per (token, head): the parts of the token's keys added up in their order
__global__ void __launch_bounds__(128)
latent_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, const int* __restrict__ token_req,
                    const float* __restrict__ sink, const __nv_bfloat16* __restrict__ gate, long long gate_tok,
                    __nv_bfloat16* __restrict__ out, long long o_tok, long long o_head, int H, int R, int groups, int n_splits) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    const int n = blockIdx.x, h = blockIdx.y;
    if (token_req[n] < 0) return;
    const int g = h / kRows, row = h % kRows;
    const size_t item0 = ((size_t)n * groups + g) * n_splits;
    float m = sink ? sink[h] * kLog2e : -INFINITY;
    for (int s = 0; s < n_splits; ++s) m = fmaxf(m, part_ml[((item0 + s) * kRows + row) * 2]);
    float l = sink ? ns_exp2(sink[h] * kLog2e - m) : 0.f;
    for (int s = 0; s < n_splits; ++s) {
        const float* ml = part_ml + ((item0 + s) * kRows + row) * 2;
        l += ml[1] * ns_exp2(ml[0] - m);  // an empty part left (-inf, 0)
    }
    float f = 1.f / l;
    if (gate) f *= 1.f / (1.f + expf(-__bfloat162float(gate[(size_t)n * gate_tok + h])));
    for (int e = threadIdx.x; e < R; e += blockDim.x) {
        float a = 0.f;
        for (int s = 0; s < n_splits; ++s)
            a += part_o[((item0 + s) * kRows + row) * R + e] * ns_exp2(part_ml[((item0 + s) * kRows + row) * 2] - m);
        out[(size_t)n * o_tok + (size_t)h * o_head + e] = __float2bfloat16_rn(a * f);
    }
}

}  // namespace

// As ns_attention_latent, bfloat16 only.  n_splits > 1: part_o [tokens * head groups * n_splits * 16 * R] and part_ml
// [tokens * head groups * n_splits * 16 * 2] float scratch, head groups = ceil(H / 16).
NS_API int ns_attention_latent_tc(const void* q_lat, long long ql_tok, long long ql_head, const void* q_rot, long long qr_tok,
                                  long long qr_head, const void* cache, const int* block_table, int table_stride,
                                  const int* token_req, const int* positions, const float* sink, const void* gate,
                                  long long gate_tok, void* out, long long o_tok, long long o_head, float* part_o, float* part_ml,
                                  int n_tokens, int H, int R, int r, int page_size, float scale, int window, int n_splits,
                                  cudaStream_t stream) {
    if (n_tokens <= 0) return NS_OK;
    if (R % 16 || r % 16 || R < 16 || R > 512)
        NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_latent_tc: a latent of %d and a rotated part of %d features (multiples of 16, the latent at most 512)", R, r);
    if (o_tok % 2 || o_head % 2 || ((uintptr_t)out & 3) || ((uintptr_t)cache & 15))
        NS_FAIL(NS_ERR_ARGUMENT, "ns_attention_latent_tc: the output's strides must be even and the cache 16-byte aligned");
    if (n_splits < 1 || n_splits > 64 || (n_splits > 1 && (!part_o || !part_ml))) NS_FAIL(NS_ERR_ARGUMENT, "ns_attention_latent_tc: n_splits=%d", n_splits);
    const int D = R + r, groups = (H + kRows - 1) / kRows;
    const size_t smem = ((size_t)(kKeysTile + kRows) * (D + 8) + 2 * kRows * kPStride) * sizeof(__nv_bfloat16) + 2 * kWarps * kRows * sizeof(float);
    dim3 grid(n_tokens, groups, n_splits);
    const int units = (R / 16 + kWarps - 1) / kWarps;
#define NS_LATENT_TC(U)                                                                                                        \
    {                                                                                                                          \
        if (smem > 48 * 1024)                                                                                                  \
            NS_CUDA(cudaFuncSetAttribute(attention_latent_tc_kernel<U>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        NS_LAUNCH((attention_latent_tc_kernel<U>), grid, kWarps * 32, smem, stream, (const __nv_bfloat16*)q_lat, ql_tok, ql_head,        \
                  (const __nv_bfloat16*)q_rot, qr_tok, qr_head, (const __nv_bfloat16*)cache, block_table, table_stride, token_req, \
                  positions, sink, (const __nv_bfloat16*)gate, gate_tok, (__nv_bfloat16*)out, o_tok, o_head, part_o, part_ml, H, R, \
                  r, page_size, scale, window, n_splits);                                                                       \
    }
    if (units <= 1) NS_LATENT_TC(1)
    else if (units <= 2) NS_LATENT_TC(2)
    else NS_LATENT_TC(4)
#undef NS_LATENT_TC
    NS_CHECK_LAUNCH("ns_attention_latent_tc");
    if (n_splits > 1) {
        NS_LAUNCH(latent_merge_kernel, dim3(n_tokens, H), 128, 0, stream, (const float*)part_o, (const float*)part_ml, token_req, sink,
                  (const __nv_bfloat16*)gate, gate_tok, (__nv_bfloat16*)out, o_tok, o_head, H, R, groups, n_splits);
        NS_CHECK_LAUNCH("ns_latent_merge");
    }
    return NS_OK;
}

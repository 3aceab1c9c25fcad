// Routed experts on the tensor cores for steps of up to a few hundred tokens, without a host round trip.
//
// ns_moe_plan has laid the (token, choice) pairs out so that every expert's pairs are neighbours: offsets[e] ..
// offsets[e + 1] are the rows of expert e, pair_of[row] the pair that sits there.  A block takes one expert and a slice of
// its features, reads how many rows the expert has from `offsets` on the device, and multiplies those rows (32 at a time,
// two m16n8k16 row tiles) with its slice of the expert's weights, which stream through shared memory in chunks of 64
// along k, double-buffered with cp.async.  Two products:
//   gated   act[row, f] = silu(x[token(row)] . gate_e[f]) * (x[token(row)] . up_e[f])      64 features a block, A rows gathered
//   plain   y[row, i]   = act[row] . down_e[i]                                                128 features a block
// Each weight is read once per 32 rows of its expert, so a decode step of many requests reads every chosen expert once
// instead of once per (token, choice).  bfloat16, k a multiple of 8.
#include "mma_utils.cuh"

namespace {

constexpr int kChunkK = 64, kTileW = 128, kStride = kChunkK + 8;

// MT: row tiles of 16 per pass (2 for steps of a few tokens per expert, 4 for prompts: twice the products per weight fragment)
template <bool GATED, int MT>
__global__ void __launch_bounds__(128)
moe_grouped_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const int* __restrict__ pair_of, int top,
                   const int* __restrict__ offsets, const __nv_bfloat16* __restrict__ w_a, const __nv_bfloat16* __restrict__ w_b,
                   __nv_bfloat16* __restrict__ out, long long ldo, int F, int K) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    constexpr int kTileM = 16 * MT;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [2][16 MT][72]
    __nv_bfloat16* ws = xs + 2 * kTileM * kStride;                    // [2][128][72]
    const int e = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int off = offsets[e], count = offsets[e + 1] - off;
    if (count <= 0) return;
    constexpr int kFeat = GATED ? 64 : 128;
    const int f0 = blockIdx.y * kFeat;
    const int piece = tid & 7, lrow = tid >> 3;  // this thread's 16-byte piece of a chunk's row, and its first row

    // the weight rows this thread copies: rows lrow + 16 i of the block's 128
    const __nv_bfloat16* wp[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int row = lrow + 16 * i;
        const int f = GATED ? f0 + (row & 63) : f0 + row;
        const __nv_bfloat16* base = (GATED && row >= 64) ? w_b : w_a;
        wp[i] = f < F ? base + ((size_t)e * F + f) * K : nullptr;
    }
    const int rbA = GATED ? 16 * warp : 32 * warp, rbB = GATED ? 64 + 16 * warp : 32 * warp + 16;
    const int n_chunks = (K + kChunkK - 1) / kChunkK;

    for (int m0 = 0; m0 < count; m0 += kTileM) {
        const __nv_bfloat16* xp[MT];
#pragma unroll
        for (int i = 0; i < MT; ++i) {
            const int m = m0 + lrow + 16 * i;
            if (m < count) {
                const int row = off + m;
                xp[i] = x + (size_t)(GATED ? pair_of[row] / top : row) * ldx;
            } else {
                xp[i] = nullptr;
            }
        }
        float acc[MT][4][4];
#pragma unroll
        for (int a = 0; a < MT; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[a][b][c] = 0.f;

        auto load = [&](int chunk, int buf) {
            const int k = chunk * kChunkK + piece * 8;
            const bool in_k = k < K;
#pragma unroll
            for (int i = 0; i < MT; ++i)
                ns_cp_async16(xs + (buf * kTileM + lrow + 16 * i) * kStride + piece * 8, xp[i] && in_k ? xp[i] + k : x, xp[i] && in_k);
#pragma unroll
            for (int i = 0; i < 8; ++i)
                ns_cp_async16(ws + (buf * kTileW + lrow + 16 * i) * kStride + piece * 8, wp[i] && in_k ? wp[i] + k : w_a, wp[i] && in_k);
            ns_cp_async_commit();
        };
        __syncthreads();  // the buffers of the pass before have been read
        load(0, 0);
        for (int c = 0; c < n_chunks; ++c) {
            const int buf = c & 1;
            if (c + 1 < n_chunks) {
                load(c + 1, buf ^ 1);
                ns_cp_async_wait<1>();
            } else {
                ns_cp_async_wait<0>();
            }
            __syncthreads();
            const __nv_bfloat16* xb = xs + buf * kTileM * kStride;
            const __nv_bfloat16* wb = ws + buf * kTileW * kStride;
#pragma unroll
            for (int kk = 0; kk < kChunkK / 16; ++kk) {
                uint32_t bA[4], bB[4];
                const int arow = (lane & 7) + ((lane >> 3) & 1) * 8, acol = kk * 16 + (lane >> 4) * 8;
                const int brow = (lane & 7) + (lane >> 4) * 8, bcol = kk * 16 + ((lane >> 3) & 1) * 8;
                ns_ldmatrix_x4(bA, wb + (rbA + brow) * kStride + bcol);
                ns_ldmatrix_x4(bB, wb + (rbB + brow) * kStride + bcol);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    uint32_t a[4];
                    ns_ldmatrix_x4(a, xb + (16 * mt + arow) * kStride + acol);
                    ns_mma_bf16(acc[mt][0], a, bA[0], bA[1]);
                    ns_mma_bf16(acc[mt][1], a, bA[2], bA[3]);
                    ns_mma_bf16(acc[mt][2], a, bB[0], bB[1]);
                    ns_mma_bf16(acc[mt][3], a, bB[2], bB[3]);
                }
            }
            __syncthreads();  // this buffer is free for the chunk after the next
        }
        // rows lane / 4 and lane / 4 + 8 of each row tile, columns (lane % 4) * 2 and the next
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int m = m0 + mt * 16 + (lane >> 2) + half * 8;
                if (m >= count) continue;
                __nv_bfloat16* orow = out + (size_t)(off + m) * ldo;
                if (GATED) {
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int f = f0 + 16 * warp + 8 * j + (lane & 3) * 2;
                        const float g0 = acc[mt][j][half * 2], g1 = acc[mt][j][half * 2 + 1];
                        const float u0 = acc[mt][j + 2][half * 2], u1 = acc[mt][j + 2][half * 2 + 1];
                        const float v0 = g0 / (1.f + __expf(-g0)) * u0, v1 = g1 / (1.f + __expf(-g1)) * u1;
                        if (f + 1 < F) *reinterpret_cast<uint32_t*>(orow + f) = ns_pack_bf16(v0, v1);
                        else if (f < F) orow[f] = __float2bfloat16_rn(v0);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int f = f0 + 32 * warp + 8 * j + (lane & 3) * 2;
                        const float v0 = acc[mt][j][half * 2], v1 = acc[mt][j][half * 2 + 1];
                        if (f + 1 < F) *reinterpret_cast<uint32_t*>(orow + f) = ns_pack_bf16(v0, v1);
                        else if (f < F) orow[f] = __float2bfloat16_rn(v0);
                    }
                }
            }
    }
}

}  // namespace

// x [tokens, width]; pair_of, offsets from ns_moe_plan; w_gate, w_up [E, ff, width]; w_down [E, width, ff];
// act [pairs, ff] and ys [pairs, width] in the plan's row order; everything bfloat16, width and ff multiples of 8.
// rows_per_expert: the step's pairs over the experts (the host's guess of how many rows an expert holds).
NS_API int ns_moe_grouped(const void* x, const int* pair_of, const int* offsets, const void* w_gate, const void* w_up,
                          const void* w_down, void* act, void* ys, int n_experts, int top, int width, int ff, int rows_per_expert,
                          cudaStream_t stream) {
    if (width % 8 || ff % 8) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_moe_grouped: width %d and expert width %d must be multiples of 8", width, ff);
    if ((((uintptr_t)x | (uintptr_t)w_gate | (uintptr_t)w_up | (uintptr_t)w_down | (uintptr_t)act) % 16) || ((uintptr_t)ys % 4))
        NS_FAIL(NS_ERR_ARGUMENT, "ns_moe_grouped: operands must start on 16 bytes");
    // row tiles per pass: prompts, whose experts hold dozens of rows each, take passes of 64 rows
    const bool wide = rows_per_expert >= 48;
    const size_t smem = (size_t)2 * ((wide ? 64 : 32) + kTileW) * kStride * sizeof(__nv_bfloat16);
    const dim3 grid_a(n_experts, (ff + 63) / 64), grid_b(n_experts, (width + 127) / 128);
#define NS_GROUPED(MT)                                                                                                              \
    {                                                                                                                               \
        if (smem > 48 * 1024) {                                                                                                     \
            NS_CUDA(cudaFuncSetAttribute(moe_grouped_kernel<true, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));      \
            NS_CUDA(cudaFuncSetAttribute(moe_grouped_kernel<false, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));     \
        }                                                                                                                           \
        NS_LAUNCH((moe_grouped_kernel<true, MT>), grid_a, 128, smem, stream, (const __nv_bfloat16*)x, (long long)width, pair_of, top,  \
                  offsets, (const __nv_bfloat16*)w_gate, (const __nv_bfloat16*)w_up, (__nv_bfloat16*)act, (long long)ff, ff, width);   \
        NS_CHECK_LAUNCH("ns_moe_grouped");                                                                                          \
        NS_LAUNCH((moe_grouped_kernel<false, MT>), grid_b, 128, smem, stream, (const __nv_bfloat16*)act, (long long)ff, pair_of, top, \
                  offsets, (const __nv_bfloat16*)w_down, (const __nv_bfloat16*)nullptr, (__nv_bfloat16*)ys, (long long)width, width, ff); \
        NS_CHECK_LAUNCH("ns_moe_grouped");                                                                                          \
    }
    if (wide) NS_GROUPED(4) else NS_GROUPED(2)
#undef NS_GROUPED
    return NS_OK;
}

// Router of the MoE layer: logits = x . Wt^T, sigmoid, + per-expert bias, top-k, renormalised fp16 weights.
// Replaces router_k (runtime/core/exl3_router.py:21-131) for any number of rows. Unlike the reference kernel (split-K
// with fp32 atomics, fast-math exp) every logit is summed in one fixed order with correctly rounded operations, and the
// sigmoid uses a fixed polynomial exp, so the selected experts are reproducible bit for bit by the CPU checker.
//   logit[r][e]: lane L of a warp sums columns i*256 + L*8 + j (i outer, j inner) with fused multiply-adds, then five
//   butterfly steps (xor 16, 8, 4, 2, 1) add the 32 partial sums.
#include "hmoe_common.cuh"
#include "hmoe_internal.h"

namespace hmoe {
namespace {

constexpr int RW = 8;     // warps per block = experts per block
constexpr int RR = 4;     // rows per block

template <bool BF>
__device__ __forceinline__ void widen8(const uint4& v, float* f)
{
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    #pragma unroll
    for (int i = 0; i < 4; ++i)
    {
        if (BF) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
        else { const float2 t = __half22float2(*(const __half2*) &w[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
    }
}

template <bool XBF, bool WBF>
__global__ void __launch_bounds__(RW * 32) router_logits_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ wt,
                                                                int R, int H, int E, float* __restrict__ logits)
{
    extern __shared__ __align__(16) uint16_t xs[];          // [RR][H]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r0 = blockIdx.y * RR, nr = R - r0 < RR ? R - r0 : RR;
    for (int i = threadIdx.x * 8; i < RR * H; i += blockDim.x * 8)
    {
        const int r = i / H;
        *(uint4*) (xs + i) = r < nr ? *(const uint4*) (x + (size_t) (r0 + r) * H + (i % H)) : make_uint4(0, 0, 0, 0);
    }
    __syncthreads();
    const int e = blockIdx.x * RW + warp;
    if (e >= E) return;
    float acc[RR];
    #pragma unroll
    for (int r = 0; r < RR; ++r) acc[r] = 0.f;
    const uint16_t* w = wt + (size_t) e * H;
    // four 256-column steps per trip with their weight loads issued first; the additions stay in column order
    for (int k0 = lane * 8; k0 < H; k0 += 1024)
    {
        uint4 wv[4];
        #pragma unroll
        for (int u = 0; u < 4; ++u) wv[u] = k0 + u * 256 < H ? ldg128_nc(w + k0 + u * 256) : make_uint4(0, 0, 0, 0);
        #pragma unroll
        for (int u = 0; u < 4; ++u)
        {
            const int k = k0 + u * 256;
            if (k < H)
            {
                float wf[8];
                widen8<WBF>(wv[u], wf);
                #pragma unroll
                for (int r = 0; r < RR; ++r)
                {
                    float xf[8];
                    widen8<XBF>(*(const uint4*) (xs + r * H + k), xf);
                    #pragma unroll
                    for (int j = 0; j < 8; ++j) acc[r] = __fmaf_rn(xf[j], wf[j], acc[r]);
                }
            }
        }
    }
    #pragma unroll
    for (int r = 0; r < RR; ++r)
    {
        float a = acc[r];
        #pragma unroll
        for (int o = 16; o; o >>= 1) a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, o));
        if (lane == 0 && r < nr) logits[(size_t) (r0 + r) * E + e] = a;
    }
}

// one warp per row: keys, top-k rounds (max key, then lowest index holding it), weights
__global__ void __launch_bounds__(256) router_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int R, int E,
                                                         int topk, float scale, int64_t* __restrict__ sel, __half* __restrict__ rw)
{
    const int lane = threadIdx.x & 31, r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= R) return;
    unsigned key[8]; float act[8];
    #pragma unroll
    for (int i = 0; i < 8; ++i)
    {
        const int e = lane + 32 * i;
        if (e < E)
        {
            const float l = logits[(size_t) r * E + e];
            act[i] = __fdiv_rn(1.f, __fadd_rn(1.f, det_expf(-l)));
            const unsigned u = __float_as_uint(__fadd_rn(act[i], bias ? bias[e] : 0.f));
            key[i] = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
        }
        else { act[i] = 0.f; key[i] = 0u; }
    }
    float sum = 0.f, mine_w = 0.f; int mine_id = 0;
    for (int k = 0; k < topk; ++k)
    {
        unsigned lk = 0u; int li = 0;
        #pragma unroll
        for (int i = 0; i < 8; ++i) if (key[i] > lk) { lk = key[i]; li = i; }
        const unsigned m = __reduce_max_sync(0xffffffffu, lk);
        const unsigned bi = __reduce_min_sync(0xffffffffu, lk == m ? (unsigned) (lane + 32 * li) : 0xffffffffu);
        float a = 0.f;
        if ((int) (bi & 31) == lane)
        {
            #pragma unroll
            for (int i = 0; i < 8; ++i) if (i == (int) (bi >> 5)) { a = act[i]; key[i] = 0u; }
        }
        a = __shfl_sync(0xffffffffu, a, bi & 31);
        sum = __fadd_rn(sum, a);
        if (lane == k) { mine_w = a; mine_id = (int) bi; }
    }
    if (lane < topk)
    {
        sel[(size_t) r * topk + lane] = mine_id;
        rw[(size_t) r * topk + lane] = __float2half_rn(__fdiv_rn(__fmul_rn(mine_w, scale), __fadd_rn(sum, 1e-20f)));
    }
}

}  // namespace

size_t router_ws_bytes(int R, int E) { return ((size_t) R * E * 4 + 255) / 256 * 256; }

int router_launch(const void* x, int x_dtype, const void* wt, int w_dtype, const float* bias, int R, int H, int E, int topk,
                  float scale, int64_t* sel, void* rw, void* ws, size_t ws_bytes, cudaStream_t st)
{
    if (R < 1 || E < 32 || E > 256 || E % 32 || H % 256 || H < 256 || topk < 1 || topk > TOPK_MAX || topk > E)
        return fail(HMOE_E_ARG, "hmoe_router: needs R >= 1, E % 32 == 0, E <= 256, H % 256 == 0, topk <= 8");
    if ((x_dtype != HMOE_F16 && x_dtype != HMOE_BF16) || (w_dtype != HMOE_F16 && w_dtype != HMOE_BF16))
        return fail(HMOE_E_ARG, "hmoe_router: x and wt must be fp16 or bf16");
    if (!x || !wt || !sel || !rw || !ws) return fail(HMOE_E_ARG, "hmoe_router: null pointer");
    if (ws_bytes < router_ws_bytes(R, E)) return fail(HMOE_E_WS, "hmoe_router: workspace too small");
    const size_t smem = (size_t) RR * H * 2;
    if (smem > 200 * 1024) return fail(HMOE_E_ARG, "hmoe_router: H too large");
    const dim3 grid((E + RW - 1) / RW, (R + RR - 1) / RR);
    float* logits = (float*) ws;
    const uint16_t* xp = (const uint16_t*) x; const uint16_t* wp = (const uint16_t*) wt;
    static bool attr = false;
    if (!attr)
    {
        cudaFuncSetAttribute(router_logits_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(router_logits_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(router_logits_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(router_logits_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        attr = true;
    }
    const bool xb = x_dtype == HMOE_BF16, wb = w_dtype == HMOE_BF16;
    if (!xb && !wb) router_logits_kernel<false, false><<<grid, RW * 32, smem, st>>>(xp, wp, R, H, E, logits);
    else if (!xb && wb) router_logits_kernel<false, true><<<grid, RW * 32, smem, st>>>(xp, wp, R, H, E, logits);
    else if (xb && !wb) router_logits_kernel<true, false><<<grid, RW * 32, smem, st>>>(xp, wp, R, H, E, logits);
    else router_logits_kernel<true, true><<<grid, RW * 32, smem, st>>>(xp, wp, R, H, E, logits);
    router_topk_kernel<<<(R + 7) / 8, 256, 0, st>>>(logits, bias, R, E, topk, scale, sel, (__half*) rw);
    count_launches(2);
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return fail(HMOE_E_CUDA, cudaGetErrorString(err));
    return HMOE_OK;
}

}  // namespace hmoe

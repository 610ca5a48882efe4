// The shared expert in the reference's own format: int8 codes (value = code - 128) with one fp32 scale per output row, stored
// in the dense GEMV fragment order of its int8 linears (runtime/core/hecate_runtime.py:38-48, docker/patches/exllamav3/fold/
// dense_i8.cu:1-8): for W[N][K], groups of 64 rows (4 strips of 16), blocks of 32 columns,
//   byte ((((((((gr * K/32 + kb) * 4 + s) * 8 + g) * 4 + q) * 2 + t) * 2 + h) * 2 + c) * 2 + rh
// holds row gr*64 + s*16 + rh*8 + g, column kb*32 + t*16 + h*8 + q*2 + c: per lane (g, q) and strip 16 bytes = the m16n8k16
// A fragments of two 16-column steps. A 2 KB unit is 64 rows x 32 columns.
//
// The reference runs this expert inside moe4 as one more slot (runtime/tier/tier_split.py:495-514,553-568;
// runtime/tier/moe4/moe4.cu:435-440,490-505). Here it is a pair of small kernels beside the routed experts' streaming
// kernels, because it is 2 % of a step's bytes: every warp takes a contiguous range of units straight from global memory
// (all of a unit's loads issued before the first is used, the next unit's loads in flight during the MMAs), multiplies them
// with all rows of the step (two 8-column MMA tiles), and adds its partial sums with fp32 reductions:
//   gate_up -> Gs[row][gate | up][I]   (rows R*topk .. of the per-pick buffer the prepare kernel zeroes)
//   down    -> y[row][H], the operand SiLU(gate) * up computed from Gs on the fly (weight 1)
// Per-row scales are applied to the partial sums as they leave. Rows outside the step (>= R) and, under expert parallelism,
// rows of other ranks (r % shared_mod != shared_rem) are computed as zeros and not written.
#include "hmoe_common.cuh"
#include "hmoe_internal.h"

namespace hmoe {
namespace {

constexpr int SW = 16, STHREADS = SW * 32;

// 4 bytes (c0 rh0, c0 rh1, c1 rh0, c1 rh1) -> fp16x2 (row g: c0, c1) and (row g + 8: c0, c1), value code - 128, exactly
__device__ __forceinline__ void dec_i8(uint32_t w, uint32_t& lo, uint32_t& hi)
{
    uint32_t h0, h1;
    asm("lop3.b32 %0, %1, 0x00ff00ff, 0x64006400, 0xea;" : "=r"(h0) : "r"(w));
    asm("lop3.b32 %0, %1, 0x00ff00ff, 0x64006400, 0xea;" : "=r"(h1) : "r"(w >> 8));
    asm("sub.f16x2 %0, %1, %2;" : "=r"(lo) : "r"(h0), "r"(0x64806480u));
    asm("sub.f16x2 %0, %1, %2;" : "=r"(hi) : "r"(h1), "r"(0x64806480u));
}
__device__ __forceinline__ void red_add_f32(float* p, float v)
{
    asm volatile("red.global.add.f32 [%0], %1;" ::"l"(__cvta_generic_to_global(p)), "f"(v) : "memory");
}

struct SharedArgs
{
    int H, I, R, sh_mod, sh_rem;
    const uint4* gate_w; const uint4* up_w; const uint4* down_w;     // int8, fragment order
    const float* gate_s; const float* up_s; const float* down_s;    // fp32 per output row
    const __half* xf;         // [16][H] the step's rows in the MMA column order (prepare kernel)
    float* gs;                // [16][2][I] gate and up sums of the shared expert
    float* y;                 // [R][H]
    const unsigned* gen_ptr; size_t slot_stride;
};

// One unit against the two row tiles. w[s] = the lane's 16 bytes of strip s; b[j][2t + h] = operand words of row tile j.
__device__ __forceinline__ void unit_mma(const uint4 (&w)[4], const uint32_t (&b)[2][4], float (&acc)[4][2][4])
{
    #pragma unroll
    for (int s = 0; s < 4; ++s)
    {
        const uint32_t ww[4] = {w[s].x, w[s].y, w[s].z, w[s].w};
        #pragma unroll
        for (int t = 0; t < 2; ++t)
        {
            uint32_t a[4];
            dec_i8(ww[2 * t], a[0], a[1]);
            dec_i8(ww[2 * t + 1], a[2], a[3]);
            #pragma unroll
            for (int j = 0; j < 2; ++j) mma_f16(acc[s][j], a, b[j][2 * t], b[j][2 * t + 1]);
        }
    }
}

// DOWN = false: units of gate then up, (matrix, 64-row group, 32-column block) with the block fastest. DOWN = true: units of down.
template <bool DOWN>
__global__ void __launch_bounds__(STHREADS) shared_i8_kernel(const SharedArgs a)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
    const int K = DOWN ? a.I : a.H, N = DOWN ? a.H : a.I, KB = K / 32, NG = N / 64;
    const long long total = (long long) (DOWN ? 1 : 2) * NG * KB;
    const long long nw = (long long) gridDim.x * SW, wid = (long long) blockIdx.x * SW + warp;
    long long u = total * wid / nw;
    const long long u1 = total * (wid + 1) / nw;
    if (u >= u1) return;
    float* const yout = DOWN ? a.y + (a.gen_ptr ? (size_t) (*a.gen_ptr & 1u) * a.slot_stride : 0) : nullptr;
    // rows of the two tiles this lane feeds (operand) and receives (results: tile columns 2q, 2q + 1)
    bool live_b[2], live_c[2][2];
    #pragma unroll
    for (int j = 0; j < 2; ++j)
    {
        const int rb = 8 * j + g;
        live_b[j] = rb < a.R && rb % a.sh_mod == a.sh_rem;
        #pragma unroll
        for (int c = 0; c < 2; ++c) { const int rc = 8 * j + 2 * q + c; live_c[j][c] = rc < a.R && rc % a.sh_mod == a.sh_rem; }
    }
    auto load_w = [&](long long uu, uint4 (&w)[4]) {
        const int kb = (int) (uu % KB), row = (int) (uu / KB);            // row = matrix * NG + 64-row group
        const uint4* base = DOWN ? a.down_w : (row >= NG ? a.up_w : a.gate_w);
        const uint4* p = base + ((size_t) (row % NG) * KB + kb) * 128 + lane;
        #pragma unroll
        for (int s = 0; s < 4; ++s) w[s] = ldg128_nc(p + s * 32);
    };
    auto load_b = [&](long long uu, uint32_t (&b)[2][4]) {
        const int kb = (int) (uu % KB);
        #pragma unroll
        for (int j = 0; j < 2; ++j)
        {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (live_b[j])
            {
                if (!DOWN) v = ldg128((const char*) (a.xf + (size_t) (8 * j + g) * a.H) + (kb >> 1) * 128 + q * 32 + (kb & 1) * 16);
                else
                {
                    // SiLU(gate) * up of columns kb*32 + 16 t + 8 h + 2 q (+ 1), from the sums the first launch left
                    const float* gp = a.gs + (size_t) (8 * j + g) * 2 * a.I + kb * 32 + 2 * q;
                    uint32_t wv[4];
                    #pragma unroll
                    for (int i = 0; i < 4; ++i)
                    {
                        const float2 gg = __ldcg((const float2*) (gp + (i >> 1) * 16 + (i & 1) * 8)), uu2 = __ldcg((const float2*) (gp + a.I + (i >> 1) * 16 + (i & 1) * 8));
                        const __half2 h = __floats2half2_rn(gg.x / (1.f + __expf(-gg.x)) * uu2.x, gg.y / (1.f + __expf(-gg.y)) * uu2.y);
                        wv[i] = *(const uint32_t*) &h;
                    }
                    v = make_uint4(wv[0], wv[1], wv[2], wv[3]);
                }
            }
            b[j][0] = v.x; b[j][1] = v.y; b[j][2] = v.z; b[j][3] = v.w;
        }
    };
    float acc[4][2][4];
    #pragma unroll
    for (int s = 0; s < 4; ++s)
        #pragma unroll
        for (int j = 0; j < 2; ++j) acc[s][j][0] = acc[s][j][1] = acc[s][j][2] = acc[s][j][3] = 0.f;
    auto flush = [&](int row) {                                       // row = matrix * NG + 64-row group of the finished sums
        const int mat = row >= NG ? 1 : 0, gr = row % NG;
        const float* sc = (DOWN ? a.down_s : (mat ? a.up_s : a.gate_s)) + gr * 64 + g;
        #pragma unroll
        for (int s = 0; s < 4; ++s)
        {
            const float s0 = __ldg(sc + s * 16), s1 = __ldg(sc + s * 16 + 8);
            #pragma unroll
            for (int j = 0; j < 2; ++j)
                #pragma unroll
                for (int c = 0; c < 2; ++c)
                {
                    if (live_c[j][c])
                    {
                        const int r = 8 * j + 2 * q + c;
                        float* dst = DOWN ? yout + (size_t) r * a.H + gr * 64 + s * 16 + g
                                          : a.gs + (size_t) r * 2 * a.I + (size_t) mat * a.I + gr * 64 + s * 16 + g;
                        red_add_f32(dst, acc[s][j][c] * s0);
                        red_add_f32(dst + 8, acc[s][j][2 + c] * s1);
                    }
                    acc[s][j][c] = 0.f; acc[s][j][2 + c] = 0.f;
                }
        }
    };
    uint4 w[4], wn[4];
    uint32_t b[2][4], bn[2][4];
    load_w(u, w); load_b(u, b);
    for (; u < u1; ++u)
    {
        const bool more = u + 1 < u1;
        if (more) { load_w(u + 1, wn); load_b(u + 1, bn); }
        unit_mma(w, b, acc);
        if (!more || (u + 1) % KB == 0) flush((int) (u / KB));
        if (more)
        {
            #pragma unroll
            for (int s = 0; s < 4; ++s) w[s] = wn[s];
            #pragma unroll
            for (int j = 0; j < 2; ++j)
                #pragma unroll
                for (int i = 0; i < 4; ++i) b[j][i] = bn[j][i];
        }
    }
}

}  // namespace

// gs: device buffer of at least 16 * 2 * I floats, zero on entry (the prepare kernel's cleared region)
int shared_i8_launch(const hmoe_layer* L, int R, int sh_mod, int sh_rem, const __half* xf, float* gs, float* y, const unsigned* gen_ptr,
                     size_t slot_stride, int sms, cudaStream_t st)
{
    if (L->H % 64 || L->I % 64) return fail(HMOE_E_ARG, "hmoe_decode: int8 shared expert needs H and I to be multiples of 64");
    SharedArgs a;
    a.H = L->H; a.I = L->I; a.R = R; a.sh_mod = sh_mod; a.sh_rem = sh_rem;
    a.gate_w = (const uint4*) L->sh_gate_w; a.up_w = (const uint4*) L->sh_up_w; a.down_w = (const uint4*) L->sh_down_w;
    a.gate_s = (const float*) L->sh_gate_s; a.up_s = (const float*) L->sh_up_s; a.down_s = (const float*) L->sh_down_s;
    a.xf = xf; a.gs = gs; a.y = y; a.gen_ptr = gen_ptr; a.slot_stride = slot_stride;
    shared_i8_kernel<false><<<sms, STHREADS, 0, st>>>(a);
    shared_i8_kernel<true><<<sms, STHREADS, 0, st>>>(a);
    count_launches(2);
    return HMOE_OK;
}

}  // namespace hmoe

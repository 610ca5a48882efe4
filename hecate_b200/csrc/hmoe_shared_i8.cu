// The shared expert in the reference's own format: int8 codes (value = code - 128) with one fp32 scale per output row, stored
// in the dense GEMV fragment order of its int8 linears (runtime/core/hecate_runtime.py:38-48, docker/patches/exllamav3/fold/
// dense_i8.cu:1-8): for W[N][K], groups of 64 rows (4 strips of 16), blocks of 32 columns,
//   byte ((((((((gr * K/32 + kb) * 4 + s) * 8 + g) * 4 + q) * 2 + t) * 2 + h) * 2 + c) * 2 + rh
// holds row gr*64 + s*16 + rh*8 + g, column kb*32 + t*16 + h*8 + q*2 + c: per lane (g, q) and strip 16 bytes = the m16n8k16
// A fragments of two 16-column steps. A 2 KB unit is 64 rows x 32 columns.
//
// The reference runs this expert inside moe4 as one more slot (runtime/tier/tier_split.py:495-514,553-568;
// runtime/tier/moe4/moe4.cu:435-440,490-505). Here it is a pair of small kernels beside the routed experts' streaming
// kernels, because it is 2 % of a step's bytes: every block takes a contiguous range of units straight from global memory,
// its warps in turn (all of a unit's loads issued before the first is used, the next unit's loads in flight during the MMAs),
// multiplies them with all rows of the step (two 8-column MMA tiles), sums the warps' partial tiles through shared memory
// and adds the result with fp32 reductions:
//   gate_up -> Gs[row][gate | up][I]   (rows R*topk .. of the per-pick buffer the prepare kernel zeroes)
//   down    -> y[row][H], the operand SiLU(gate) * up computed from Gs on the fly (weight 1)
// Per-row scales are applied to the partial sums as they leave. Rows outside the step (>= R) and, under expert parallelism,
// rows of other ranks (r % shared_mod != shared_rem) are computed as zeros and not written.
#include "hmoe_common.cuh"
#include "hmoe_internal.h"

namespace hmoe {
namespace {

constexpr int SW = 16, STHREADS = SW * 32, PART = 16 * 65;

// programmatic dependent launch: let the next kernel's blocks start as this one's retire / wait for the kernel before
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
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
// A block takes a contiguous range of units and deals them to its warps in turn, so all warps are in the same 64-row group at
// the same time; where the range leaves a row group (and at its end) the warps' partial tiles are summed through shared memory
// and one set of reductions leaves the block.
template <bool DOWN>
__global__ void __launch_bounds__(STHREADS, 1) shared_i8_kernel(const SharedArgs a)
{
    extern __shared__ float part[];                       // [SW][16 tile columns][64 rows + 1]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
    const int K = DOWN ? a.I : a.H, N = DOWN ? a.H : a.I, KB = K / 32, NG = N / 64;
    const long long total = (long long) (DOWN ? 1 : 2) * NG * KB;
    const long long U0 = total * blockIdx.x / gridDim.x, U1 = total * (blockIdx.x + 1) / gridDim.x;
    float* const yout = DOWN ? a.y + (a.gen_ptr ? (size_t) (*a.gen_ptr & 1u) * a.slot_stride : 0) : nullptr;     // gen: written two kernels back
    // rows of the two tiles this lane feeds (operand)
    bool live_b[2];
    #pragma unroll
    for (int j = 0; j < 2; ++j) { const int rb = 8 * j + g; live_b[j] = rb < a.R && rb % a.sh_mod == a.sh_rem; }
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
    // the block's range, one 64-row group (segment) at a time
    bool waited = false;
    for (long long seg0 = U0; seg0 < U1;)
    {
        const int row = (int) (seg0 / KB);
        const long long seg1 = (long long) (row + 1) * KB < U1 ? (long long) (row + 1) * KB : U1;
        long long u = seg0 + warp;
        // the segment's row scale of this thread's output column (the same for all of its outputs: they are 512 apart), requested
        // now so that its latency is spent under the units and not in front of the reductions
        const float sc_n = __ldg((DOWN ? a.down_s : (row >= NG ? a.up_s : a.gate_s)) + (row % NG) * 64 + (threadIdx.x & 63));
        uint4 w[4], wn[4];
        uint32_t b[2][4], bn[2][4];
        if (u < seg1) load_w(u, w);              // weights do not depend on the kernel before: requested while it drains
        // dependents are released only after this kernel's own wait (see decode_stream_kernel: what a dependent reads before
        // its wait is then at least two completed kernels old)
        if (!waited) { pdl_wait(); pdl_launch_dependents(); waited = true; }
        if (u < seg1) load_b(u, b);
        for (; u < seg1; u += SW)
        {
            const bool more = u + SW < seg1;
            if (more) { load_w(u + SW, wn); load_b(u + SW, bn); }
            unit_mma(w, b, acc);
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
        // partial tile of this warp -> shared memory [tile column][row of the group, padded to 65], then one sum per output element
        float* mine = part + warp * PART;
        #pragma unroll
        for (int s = 0; s < 4; ++s)
            #pragma unroll
            for (int j = 0; j < 2; ++j)
            {
                #pragma unroll
                for (int c = 0; c < 2; ++c)
                {
                    mine[(8 * j + 2 * q + c) * 65 + s * 16 + g] = acc[s][j][c];
                    mine[(8 * j + 2 * q + c) * 65 + s * 16 + g + 8] = acc[s][j][2 + c];
                }
                acc[s][j][0] = acc[s][j][1] = acc[s][j][2] = acc[s][j][3] = 0.f;
            }
        __syncthreads();
        const int mat = row >= NG ? 1 : 0, gr = row % NG;
        for (int i = threadIdx.x; i < 1024; i += STHREADS)
        {
            const int r = i >> 6, n = i & 63;                        // tile column (row of the step), row of the group: consecutive n per warp
            if (r < a.R && r % a.sh_mod == a.sh_rem)
            {
                float v = 0.f;
                #pragma unroll
                for (int ww = 0; ww < SW; ++ww) v += part[ww * PART + r * 65 + n];
                float* dst = DOWN ? yout + (size_t) r * a.H + gr * 64 + n : a.gs + (size_t) r * 2 * a.I + (size_t) mat * a.I + gr * 64 + n;
                red_add_f32(dst, v * sc_n);
            }
        }
        __syncthreads();
        seg0 = seg1;
    }
    if (!waited) { pdl_wait(); pdl_launch_dependents(); }       // a block without units still orders the chain
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
    // one block of sixteen warps per SM; both launches are programmatic dependents of the kernel before them
    static DeviceOnce once;
    const size_t smem = (size_t) SW * PART * 4;
    if (once.first())
    {
        cudaFuncSetAttribute(shared_i8_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem);
        cudaFuncSetAttribute(shared_i8_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sms); cfg.blockDim = dim3(STHREADS); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, shared_i8_kernel<false>, a);
    cudaLaunchKernelEx(&cfg, shared_i8_kernel<true>, a);
    count_launches(2);
    return HMOE_OK;
}

}  // namespace hmoe

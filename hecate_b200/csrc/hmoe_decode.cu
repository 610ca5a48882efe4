// Decode path of the MoE expert layer (<= 16 rows: tokens and their MTP drafts), sm_100a.
//
// Replaces the reference's moe4 decode kernels (runtime/tier/moe4/moe4.cu:361-676: moe4_a_kernel, moe4_act_kernel,
// moe4_b_kernel and their in-kernel route()) behind the same operator surface: packed int4 experts in the reference's
// fragment order, routing as (sel, rw), fp32 output accumulated into y. Differences by design: 16 rows in one pass over
// the weights, a scale per 128 input columns (or the reference's scale per row), an int4 shared expert as one more slot.
//
// Three launches per call:
//   prepare : one block per row rewrites x as fp16 in the column order the MMAs read (optionally after the CPU engine's
//             int8 round trip), one more block builds the Route (distinct experts, their rows and weights).
//   gate_up : persistent blocks, one per SM. A work item is (slot, 64-row group of the expert's gate and up matrices);
//             items are dealt out as contiguous ranges. One producer thread streams the item's packed codes into a
//             shared-memory ring with 1-D bulk copies (16 KB gate + 16 KB up per stage, mbarrier completion); eight
//             consumer warps (four per matrix, each owning every fourth 128-column group) turn the codes into fp16 MMA
//             fragments in registers and run m16n8k16 MMAs against only the rows that picked the expert. The block then
//             reduces the eight partial tiles through shared memory, applies SiLU(g) * u * routing weight and writes the
//             result as the next kernel's MMA operand.
//   down    : same streaming structure over (64-row group of the output, slot) items, slot fastest, so that a block adds
//             every slot's contribution to a 64-column slice of y in shared memory and issues one fp32 reduction to global
//             memory per slice.
// Both streaming kernels are bound by HBM: algorithmic bytes per call are (distinct experts + shared) x the expert's
// packed size plus scales.
#include "hmoe_common.cuh"
#include "hmoe_internal.h"

namespace hmoe {

namespace {

constexpr int CW = 8;                    // consumer warps
constexpr int NTHREADS = (CW + 1) * 32;  // + one producer warp
constexpr int STAGE_BYTES = 32768;
constexpr int NSTAGE = 4;
constexpr int RED_FLOATS = 2 * 4 * 64 * 16;   // gate_up partial tiles: [matrix][k quarter][64 rows][16 columns]
constexpr int YACC_FLOATS = MAXR * 64;

struct SmemLayout
{
    static constexpr int ring = 0;
    static constexpr int red = NSTAGE * STAGE_BYTES;                  // gate_up: RED_FLOATS floats; down: YACC_FLOATS floats
    static constexpr int bars = red + RED_FLOATS * 4;                 // full[NSTAGE], empty[NSTAGE]
    static constexpr int flags = bars + 2 * NSTAGE * 8;
    static constexpr int total = flags + 16;
};

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory"); }

// ---------------------------------------------------------------------------------------------------------------------
// prepare
__global__ void __launch_bounds__(256) decode_prepare_kernel(const void* __restrict__ x, int x_bf16, const int64_t* __restrict__ sel,
    const __half* __restrict__ rw, int R, int H, int topk, int lo, int n_local, int has_shared, int act_quant,
    __half* __restrict__ xf, Route* __restrict__ route)
{
    const int tid = threadIdx.x;
    if ((int) blockIdx.x < R)
    {
        const int r = blockIdx.x;
        for (int gi = tid; gi < H / 32; gi += blockDim.x)
        {
            float v[32];
            if (x_bf16)
            {
                const uint16_t* p = (const uint16_t*) x + (size_t) r * H + gi * 32;
                #pragma unroll
                for (int k = 0; k < 32; ++k) v[k] = bf16_bits_to_float(p[k]);
            }
            else
            {
                const __half* p = (const __half*) x + (size_t) r * H + gi * 32;
                #pragma unroll
                for (int k = 0; k < 32; ++k) v[k] = __half2float(p[k]);
            }
            if (act_quant)
            {
                // the CPU engine's activation format (runtime/tier/cpuband.cpp:106-111): int8 with a scale per 32 values
                float m = 0.f;
                #pragma unroll
                for (int k = 0; k < 32; ++k) m = fmaxf(m, fabsf(v[k]));
                const float s = m > 0.f ? __fdiv_rn(m, 127.f) : 1.f;
                const float inv = __fdiv_rn(1.f, s);
                #pragma unroll
                for (int k = 0; k < 32; ++k) v[k] = __fmul_rn((float) __float2int_rn(__fmul_rn(v[k], inv)), s);
            }
            const int kb = gi >> 1, p0 = (gi & 1) * 16;
            uint32_t* dst = (uint32_t*) (xf + (size_t) r * H + kb * 64);
            #pragma unroll
            for (int p = 0; p < 16; ++p)
            {
                const __half2 h = __floats2half2_rn(v[2 * p], v[2 * p + 1]);
                dst[frag_pos(p0 + p)] = *(const uint32_t*) &h;
            }
        }
        return;
    }
    // routing block
    __shared__ int flag[256];
    __shared__ short slot_of[256];
    __shared__ int m_sh;
    for (int i = tid; i < 256; i += blockDim.x) flag[i] = 0;
    __syncthreads();
    for (int i = tid; i < R * topk; i += blockDim.x)
    {
        const int64_t e = sel[i] - lo;
        if (e >= 0 && e < n_local) flag[(int) e] = 1;
    }
    __syncthreads();
    if (tid == 0)
    {
        int m = 0;
        for (int e = 0; e < n_local; ++e) if (flag[e]) { slot_of[e] = (short) m; route->expert[m] = (short) e; ++m; }
        if (has_shared) route->expert[m] = -1;
        m_sh = m;
        route->m = m; route->nslots = m + (has_shared ? 1 : 0); route->pad = 0;
    }
    __syncthreads();
    const int m = m_sh;
    for (int j = tid; j < m + (has_shared ? 1 : 0); j += blockDim.x)
    {
        int n = 0;
        if (j < m)
        {
            const int e = route->expert[j];
            for (int r = 0; r < R; ++r)
            {
                float ws = 0.f; bool hit = false;
                for (int k = 0; k < topk; ++k)
                    if ((int) (sel[r * topk + k] - lo) == e) { ws += __half2float(rw[r * topk + k]); hit = true; }
                if (hit) { route->rows[j][n] = (unsigned char) r; route->w[j][n] = ws; ++n; }
            }
        }
        else
            for (int r = 0; r < R; ++r) { route->rows[j][n] = (unsigned char) r; route->w[j][n] = 1.f; ++n; }
        route->nrows[j] = (unsigned char) n;
        for (int i = n; i < MAXR; ++i) { route->rows[j][i] = 255; route->w[j][i] = 0.f; }
    }
    __syncthreads();
    if (tid == 0)
    {
        int t = 0;
        for (int j = 0; j < m + (has_shared ? 1 : 0); ++j) { route->tile0[j] = (short) t; t += (route->nrows[j] + 7) / 8; }
        route->ntiles = t;
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// One consumer warp's share of one ring stage: `nkb` (1 or 2) 64-column blocks of a 64-row group, i.e. one 128-column
// scale group. wsm = shared address of the warp's first 2 KB unit; xrow[nt] = this lane's activation row for tile nt
// (already offset to the first of the blocks and to the lane's 32-byte chunk). Adds into acc[strip][nt][4].
template <int NT, bool GROUPED>
__device__ __forceinline__ void consume_group(uint32_t wsm, int nkb, const char* const* xrow, const uint16_t* sc, int sc_ok,
                                              float (*acc)[NT][4], int lane)
{
    float part[4][NT][4];
    uint16_t sb[8];
    if (GROUPED)
    {
        // scales of rows strip*16 + g and + 8 for this 128-column group (bf16)
        #pragma unroll
        for (int s = 0; s < 4; ++s) { sb[2 * s] = sc_ok ? __ldg(sc + s * 16) : (uint16_t) 0; sb[2 * s + 1] = sc_ok ? __ldg(sc + s * 16 + 8) : (uint16_t) 0; }
        #pragma unroll
        for (int s = 0; s < 4; ++s)
            #pragma unroll
            for (int nt = 0; nt < NT; ++nt)
                #pragma unroll
                for (int i = 0; i < 4; ++i) part[s][nt][i] = 0.f;
    }
    for (int kbi = 0; kbi < nkb; ++kbi)
    {
        uint4 w4[4];
        #pragma unroll
        for (int s = 0; s < 4; ++s) w4[s] = lds128(wsm + kbi * 2048 + s * 512 + lane * 16);
        uint32_t bx[NT][8];
        #pragma unroll
        for (int nt = 0; nt < NT; ++nt)
        {
            const uint4 b0 = ldg128(xrow[nt] + kbi * 128), b1 = ldg128(xrow[nt] + kbi * 128 + 16);
            bx[nt][0] = b0.x; bx[nt][1] = b0.y; bx[nt][2] = b0.z; bx[nt][3] = b0.w;
            bx[nt][4] = b1.x; bx[nt][5] = b1.y; bx[nt][6] = b1.z; bx[nt][7] = b1.w;
        }
        #pragma unroll
        for (int s = 0; s < 4; ++s)
        {
            const uint32_t ww[4] = {w4[s].x, w4[s].y, w4[s].z, w4[s].w};
            #pragma unroll
            for (int t = 0; t < 4; ++t)
            {
                uint32_t a[4];
                frag_from_codes(ww[t], a);
                #pragma unroll
                for (int nt = 0; nt < NT; ++nt)
                    mma_f16(GROUPED ? part[s][nt] : acc[s][nt], a, bx[nt][2 * t], bx[nt][2 * t + 1]);
            }
        }
    }
    if (GROUPED)
    {
        #pragma unroll
        for (int s = 0; s < 4; ++s)
        {
            const float s0 = bf16_bits_to_float(sb[2 * s]), s1 = bf16_bits_to_float(sb[2 * s + 1]);
            #pragma unroll
            for (int nt = 0; nt < NT; ++nt)
            {
                acc[s][nt][0] = fmaf(s0, part[s][nt][0], acc[s][nt][0]); acc[s][nt][1] = fmaf(s0, part[s][nt][1], acc[s][nt][1]);
                acc[s][nt][2] = fmaf(s1, part[s][nt][2], acc[s][nt][2]); acc[s][nt][3] = fmaf(s1, part[s][nt][3], acc[s][nt][3]);
            }
        }
    }
}

struct DecodeArgs
{
    int H, I, group, act_quant;
    const int64_t* gate_w; const int64_t* up_w; const int64_t* down_w;
    const int64_t* gate_s; const int64_t* up_s; const int64_t* down_s;
    const void* sh_gw; const void* sh_uw; const void* sh_dw; const void* sh_gs; const void* sh_us; const void* sh_ds;
    const Route* route;
    const __half* xf;      // [R][H] prepared rows
    __half* act;           // [tiles][8][I] gate_up output = down input
    float* y;              // [R][H]
    unsigned* status;
};

// ---------------------------------------------------------------------------------------------------------------------
// gate_up
template <int NT, bool GROUPED>
__device__ __forceinline__ void gate_up_item(const DecodeArgs& a, int slot, int gr, int e, uint32_t ring, uint32_t full0, uint32_t empty0,
                                             float* red, volatile int* abort_flag, uint32_t& it, int warp, int lane)
{
    const int KB = a.H / 64, S = (KB + 7) / 8;
    const int mat = warp >> 2, kq = warp & 3, g = lane >> 2, q = lane & 3;
    const Route* rt = a.route;
    const int nrows = rt->nrows[slot];
    float acc[4][NT][4];
    #pragma unroll
    for (int s = 0; s < 4; ++s)
        #pragma unroll
        for (int nt = 0; nt < NT; ++nt)
            #pragma unroll
            for (int i = 0; i < 4; ++i) acc[s][nt][i] = 0.f;
    const char* xbase[NT];
    #pragma unroll
    for (int nt = 0; nt < NT; ++nt)
    {
        int r = rt->rows[slot][nt * 8 + g];
        if (r == 255) r = rt->rows[slot][0];
        xbase[nt] = (const char*) (a.xf + (size_t) r * a.H) + q * 32;
    }
    const uint16_t* scb = nullptr;
    if (GROUPED)
    {
        const void* sp = e >= 0 ? (const void*) (mat ? a.up_s[e] : a.gate_s[e]) : (mat ? a.sh_us : a.sh_gs);
        scb = (const uint16_t*) sp + gr * 64 + g;      // + kg * I + strip * 16 (+ 8)
    }
    for (int s = 0; s < S; ++s, ++it)
    {
        const uint32_t st = it % NSTAGE, par = (it / NSTAGE) & 1;
        if (!mbar_wait(full0 + st * 8, par, abort_flag, a.status)) return;
        const int kb = 8 * s + 2 * kq;
        if (kb < KB)
        {
            const int nkb = KB - kb < 2 ? KB - kb : 2;
            const char* xr[NT];
            #pragma unroll
            for (int nt = 0; nt < NT; ++nt) xr[nt] = xbase[nt] + kb * 128;
            consume_group<NT, GROUPED>(ring + st * STAGE_BYTES + mat * (STAGE_BYTES / 2) + 2 * kq * 2048, nkb, xr,
                                       scb + (size_t) (kb >> 1) * a.I, 1, acc, lane);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + st * 8);
    }
    // partial tiles -> shared memory: red[mat][kq][row][col], col stride CP
    constexpr int CP = 8 * NT;
    float* rp = red + (mat * 4 + kq) * 64 * CP;
    #pragma unroll
    for (int s = 0; s < 4; ++s)
        #pragma unroll
        for (int nt = 0; nt < NT; ++nt)
        {
            *(float2*) (rp + (s * 16 + g) * CP + nt * 8 + 2 * q) = make_float2(acc[s][nt][0], acc[s][nt][1]);
            *(float2*) (rp + (s * 16 + g + 8) * CP + nt * 8 + 2 * q) = make_float2(acc[s][nt][2], acc[s][nt][3]);
        }
    consumer_sync();
    // act = silu(gate) * up * routing weight; this warp handles column `warp` (+ 8) of the tile, each lane two rows
    const int n0 = 2 * lane;
    float sg0 = 1.f, sg1 = 1.f, su0 = 1.f, su1 = 1.f;
    if (!GROUPED)
    {
        const float* gsp = e >= 0 ? (const float*) a.gate_s[e] : (const float*) a.sh_gs;
        const float* usp = e >= 0 ? (const float*) a.up_s[e] : (const float*) a.sh_us;
        sg0 = __ldg(gsp + gr * 64 + n0); sg1 = __ldg(gsp + gr * 64 + n0 + 1);
        su0 = __ldg(usp + gr * 64 + n0); su1 = __ldg(usp + gr * 64 + n0 + 1);
    }
    #pragma unroll
    for (int nt = 0; nt < NT; ++nt)
    {
        const int col = nt * 8 + warp;
        float v0 = 0.f, v1 = 0.f;
        if (col < nrows)
        {
            float g0 = 0.f, g1 = 0.f, u0 = 0.f, u1 = 0.f;
            #pragma unroll
            for (int k = 0; k < 4; ++k)
            {
                g0 += red[((0 * 4 + k) * 64 + n0) * CP + col]; g1 += red[((0 * 4 + k) * 64 + n0 + 1) * CP + col];
                u0 += red[((1 * 4 + k) * 64 + n0) * CP + col]; u1 += red[((1 * 4 + k) * 64 + n0 + 1) * CP + col];
            }
            g0 *= sg0; g1 *= sg1; u0 *= su0; u1 *= su1;
            const float wr = rt->w[slot][col];
            v0 = g0 / (1.f + expf(-g0)) * u0 * wr;
            v1 = g1 / (1.f + expf(-g1)) * u1 * wr;
        }
        if (a.act_quant)
        {
            // second int8 round trip of the CPU engine (cpuband.cpp:200-207): groups of 32 consecutive outputs = 16 lanes
            float m = fmaxf(fabsf(v0), fabsf(v1));
            #pragma unroll
            for (int o = 8; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            const float s = m > 0.f ? __fdiv_rn(m, 127.f) : 1.f;
            const float inv = __fdiv_rn(1.f, s);
            v0 = __fmul_rn((float) __float2int_rn(__fmul_rn(v0, inv)), s);
            v1 = __fmul_rn((float) __float2int_rn(__fmul_rn(v1, inv)), s);
        }
        const __half2 h = __floats2half2_rn(v0, v1);
        uint32_t* dst = (uint32_t*) (a.act + ((size_t) (rt->tile0[slot] + nt) * 8 + warp) * a.I + gr * 64);
        dst[frag_pos(lane)] = *(const uint32_t*) &h;
    }
    consumer_sync();
}

template <bool GROUPED>
__global__ void __launch_bounds__(NTHREADS, 1) decode_gate_up_kernel(const DecodeArgs a)
{
    extern __shared__ __align__(1024) unsigned char smem[];
    const uint32_t sbase = smem_u32(smem);
    const uint32_t ring = sbase + SmemLayout::ring, full0 = sbase + SmemLayout::bars, empty0 = full0 + NSTAGE * 8;
    float* red = (float*) (smem + SmemLayout::red);
    volatile int* abort_flag = (volatile int*) (smem + SmemLayout::flags);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0)
    {
        for (int i = 0; i < NSTAGE; ++i) { mbar_init(full0 + i * 8, 1); mbar_init(empty0 + i * 8, CW); }
        *abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();
    const Route* rt = a.route;
    const int NG = a.I / 64, KB = a.H / 64, S = (KB + 7) / 8;
    const int P = rt->nslots * NG;
    const int p0 = (int) ((long long) P * blockIdx.x / gridDim.x), p1 = (int) ((long long) P * (blockIdx.x + 1) / gridDim.x);
    if (warp == CW)
    {
        if (lane == 0)
        {
            uint32_t it = 0;
            bool ok = true;
            for (int p = p0; p < p1 && ok; ++p)
            {
                const int slot = p / NG, gr = p % NG, e = rt->expert[slot];
                const char* gw = (const char*) (e >= 0 ? (const void*) a.gate_w[e] : a.sh_gw) + (size_t) gr * KB * 2048;
                const char* uw = (const char*) (e >= 0 ? (const void*) a.up_w[e] : a.sh_uw) + (size_t) gr * KB * 2048;
                for (int s = 0; s < S; ++s, ++it)
                {
                    const uint32_t st = it % NSTAGE;
                    if (it >= NSTAGE && !mbar_wait(empty0 + st * 8, ((it / NSTAGE) - 1) & 1, abort_flag, a.status)) { ok = false; break; }
                    const int nkb = KB - 8 * s < 8 ? KB - 8 * s : 8;
                    const uint32_t bytes = nkb * 2048;
                    mbar_expect_tx(full0 + st * 8, 2 * bytes);
                    bulk_g2s(ring + st * STAGE_BYTES, gw + (size_t) s * 16384, bytes, full0 + st * 8);
                    bulk_g2s(ring + st * STAGE_BYTES + STAGE_BYTES / 2, uw + (size_t) s * 16384, bytes, full0 + st * 8);
                }
            }
        }
    }
    else
    {
        uint32_t it = 0;
        for (int p = p0; p < p1; ++p)
        {
            const int slot = p / NG, gr = p % NG, e = rt->expert[slot];
            if (rt->nrows[slot] > 8) gate_up_item<2, GROUPED>(a, slot, gr, e, ring, full0, empty0, red, abort_flag, it, warp, lane);
            else gate_up_item<1, GROUPED>(a, slot, gr, e, ring, full0, empty0, red, abort_flag, it, warp, lane);
            if (*abort_flag) break;
        }
    }
    // Leave only when every copy this block issued has landed (a timed-out consumer may still have copies in flight):
    // the producer thread drains the stages it filled but nobody consumed.
    __syncthreads();
}

// ---------------------------------------------------------------------------------------------------------------------
// down
template <int NT, bool GROUPED>
__device__ __forceinline__ void down_item(const DecodeArgs& a, int slot, int gr, int e, uint32_t ring, uint32_t full0, uint32_t empty0,
                                          float* yacc, volatile int* abort_flag, uint32_t& it, int warp, int lane)
{
    const int KB = a.I / 64, S = (KB + 15) / 16;
    const int g = lane >> 2, q = lane & 3;
    const Route* rt = a.route;
    const int nrows = rt->nrows[slot];
    float acc[4][NT][4];
    #pragma unroll
    for (int s = 0; s < 4; ++s)
        #pragma unroll
        for (int nt = 0; nt < NT; ++nt)
            #pragma unroll
            for (int i = 0; i < 4; ++i) acc[s][nt][i] = 0.f;
    const char* xbase[NT];
    #pragma unroll
    for (int nt = 0; nt < NT; ++nt)
        xbase[nt] = (const char*) (a.act + ((size_t) (rt->tile0[slot] + nt) * 8 + g) * a.I) + q * 32;
    const uint16_t* scb = nullptr;
    if (GROUPED)
    {
        const void* sp = e >= 0 ? (const void*) a.down_s[e] : a.sh_ds;
        scb = (const uint16_t*) sp + gr * 64 + g;
    }
    for (int s = 0; s < S; ++s, ++it)
    {
        const uint32_t st = it % NSTAGE, par = (it / NSTAGE) & 1;
        if (!mbar_wait(full0 + st * 8, par, abort_flag, a.status)) return;
        const int kb = 16 * s + 2 * warp;
        if (kb < KB)
        {
            const int nkb = KB - kb < 2 ? KB - kb : 2;
            const char* xr[NT];
            #pragma unroll
            for (int nt = 0; nt < NT; ++nt) xr[nt] = xbase[nt] + kb * 128;
            consume_group<NT, GROUPED>(ring + st * STAGE_BYTES + 2 * warp * 2048, nkb, xr, scb + (size_t) (kb >> 1) * a.H, 1, acc, lane);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + st * 8);
    }
    float sd[8];
    #pragma unroll
    for (int s = 0; s < 8; ++s) sd[s] = 1.f;
    if (!GROUPED)
    {
        const float* dsp = e >= 0 ? (const float*) a.down_s[e] : (const float*) a.sh_ds;
        #pragma unroll
        for (int s = 0; s < 4; ++s) { sd[2 * s] = __ldg(dsp + gr * 64 + s * 16 + g); sd[2 * s + 1] = __ldg(dsp + gr * 64 + s * 16 + g + 8); }
    }
    // add this warp's partial (its share of the columns) into the block's slice accumulator, real row by real row
    #pragma unroll
    for (int nt = 0; nt < NT; ++nt)
        #pragma unroll
        for (int c = 0; c < 2; ++c)
        {
            const int col = nt * 8 + 2 * q + c;
            if (col < nrows)
            {
                float* yr = yacc + (int) rt->rows[slot][col] * 64;
                #pragma unroll
                for (int s = 0; s < 4; ++s)
                {
                    atomicAdd(yr + s * 16 + g, acc[s][nt][c] * sd[2 * s]);
                    atomicAdd(yr + s * 16 + g + 8, acc[s][nt][2 + c] * sd[2 * s + 1]);
                }
            }
        }
}

template <bool GROUPED>
__global__ void __launch_bounds__(NTHREADS, 1) decode_down_kernel(const DecodeArgs a, int R)
{
    extern __shared__ __align__(1024) unsigned char smem[];
    const uint32_t sbase = smem_u32(smem);
    const uint32_t ring = sbase + SmemLayout::ring, full0 = sbase + SmemLayout::bars, empty0 = full0 + NSTAGE * 8;
    float* yacc = (float*) (smem + SmemLayout::red);
    volatile int* abort_flag = (volatile int*) (smem + SmemLayout::flags);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0)
    {
        for (int i = 0; i < NSTAGE; ++i) { mbar_init(full0 + i * 8, 1); mbar_init(empty0 + i * 8, CW); }
        *abort_flag = 0;
        fence_barrier_init();
    }
    for (int i = threadIdx.x; i < YACC_FLOATS; i += blockDim.x) yacc[i] = 0.f;
    __syncthreads();
    const Route* rt = a.route;
    const int NG = a.H / 64, KB = a.I / 64, S = (KB + 15) / 16;
    const int ns = rt->nslots;
    const int P = ns * NG;
    const int p0 = (int) ((long long) P * blockIdx.x / gridDim.x), p1 = (int) ((long long) P * (blockIdx.x + 1) / gridDim.x);
    if (warp == CW)
    {
        if (lane == 0)
        {
            uint32_t it = 0;
            bool ok = true;
            for (int p = p0; p < p1 && ok; ++p)
            {
                const int gr = p / ns, slot = p % ns, e = rt->expert[slot];
                const char* dw = (const char*) (e >= 0 ? (const void*) a.down_w[e] : a.sh_dw) + (size_t) gr * KB * 2048;
                for (int s = 0; s < S; ++s, ++it)
                {
                    const uint32_t st = it % NSTAGE;
                    if (it >= NSTAGE && !mbar_wait(empty0 + st * 8, ((it / NSTAGE) - 1) & 1, abort_flag, a.status)) { ok = false; break; }
                    const int nkb = KB - 16 * s < 16 ? KB - 16 * s : 16;
                    mbar_expect_tx(full0 + st * 8, nkb * 2048);
                    bulk_g2s(ring + st * STAGE_BYTES, dw + (size_t) s * 32768, nkb * 2048, full0 + st * 8);
                }
            }
        }
    }
    else
    {
        uint32_t it = 0;
        for (int p = p0; p < p1; ++p)
        {
            const int gr = p / ns, slot = p % ns, e = rt->expert[slot];
            if (rt->nrows[slot] > 8) down_item<2, GROUPED>(a, slot, gr, e, ring, full0, empty0, yacc, abort_flag, it, warp, lane);
            else down_item<1, GROUPED>(a, slot, gr, e, ring, full0, empty0, yacc, abort_flag, it, warp, lane);
            if (*abort_flag) break;
            if (p + 1 == p1 || (p + 1) / ns != gr)
            {
                // the slice of y this block has been adding into is complete: one fp32 reduction per element to global
                consumer_sync();
                for (int i = threadIdx.x; i < R * 64; i += CW * 32)
                {
                    const float v = yacc[i];
                    if (v != 0.f) atomicAdd(a.y + (size_t) (i >> 6) * a.H + gr * 64 + (i & 63), v);
                    yacc[i] = 0.f;
                }
                consumer_sync();
            }
        }
    }
    __syncthreads();
}

}  // namespace

// ---------------------------------------------------------------------------------------------------------------------
// host side
size_t decode_ws_bytes(int H, int I)
{
    size_t b = 0;
    b += 256;                                            // status word + padding
    b += (sizeof(Route) + 255) / 256 * 256;
    b += (size_t) MAXR * H * 2;                          // xf
    b += (size_t) MAXT * 8 * I * 2;                      // act
    return (b + 255) / 256 * 256;
}

static int g_sms = 0;

int decode_launch(const hmoe_layer* L, const void* x, int x_dtype, const int64_t* sel, const void* rw, int R, int lo, int n_local,
                  int act_quant, float* y, void* ws, size_t ws_bytes, cudaStream_t st)
{
    const int H = L->H, I = L->I;
    if (R < 1 || R > MAXR) return fail(HMOE_E_ARG, "hmoe_decode: rows must be 1..16");
    if (L->topk < 1 || L->topk > TOPK_MAX) return fail(HMOE_E_ARG, "hmoe_decode: topk must be 1..8");
    if (H % 128 || I % 128 || H < 128 || I < 128) return fail(HMOE_E_ARG, "hmoe_decode: H and I must be multiples of 128");
    if (n_local < 0 || n_local > 256) return fail(HMOE_E_ARG, "hmoe_decode: at most 256 local experts");
    if (!(L->group == 0 && L->scale_dtype == HMOE_F32) && !(L->group == 128 && L->scale_dtype == HMOE_BF16))
        return fail(HMOE_E_ARG, "hmoe_decode: scales must be fp32 per row (group 0) or bf16 per 128 columns");
    if (x_dtype != HMOE_F16 && x_dtype != HMOE_BF16) return fail(HMOE_E_ARG, "hmoe_decode: x must be fp16 or bf16");
    if (ws_bytes < decode_ws_bytes(H, I)) return fail(HMOE_E_WS, "hmoe_decode: workspace too small");
    if (!x || !sel || !rw || !y || !ws) return fail(HMOE_E_ARG, "hmoe_decode: null pointer");
    if (g_sms == 0)
    {
        int dev = 0; cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
        cudaFuncSetAttribute(decode_gate_up_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemLayout::total);
        cudaFuncSetAttribute(decode_gate_up_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemLayout::total);
        cudaFuncSetAttribute(decode_down_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemLayout::total);
        cudaFuncSetAttribute(decode_down_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemLayout::total);
    }
    char* w = (char*) ws;
    unsigned* status = (unsigned*) w; w += 256;
    Route* route = (Route*) w; w += (sizeof(Route) + 255) / 256 * 256;
    __half* xf = (__half*) w; w += (size_t) MAXR * H * 2;
    __half* act = (__half*) w;
    const int has_shared = L->sh_gate_w != nullptr;
    decode_prepare_kernel<<<R + 1, 256, 0, st>>>(x, x_dtype == HMOE_BF16, sel, (const __half*) rw, R, H, L->topk, lo, n_local, has_shared,
                                                 act_quant, xf, route);
    DecodeArgs a;
    a.H = H; a.I = I; a.group = L->group; a.act_quant = act_quant;
    a.gate_w = L->gate_w; a.up_w = L->up_w; a.down_w = L->down_w; a.gate_s = L->gate_s; a.up_s = L->up_s; a.down_s = L->down_s;
    a.sh_gw = L->sh_gate_w; a.sh_uw = L->sh_up_w; a.sh_dw = L->sh_down_w; a.sh_gs = L->sh_gate_s; a.sh_us = L->sh_up_s; a.sh_ds = L->sh_down_s;
    a.route = route; a.xf = xf; a.act = act; a.y = y; a.status = status;
    const int grid = g_sms;
    if (L->group) decode_gate_up_kernel<true><<<grid, NTHREADS, SmemLayout::total, st>>>(a);
    else decode_gate_up_kernel<false><<<grid, NTHREADS, SmemLayout::total, st>>>(a);
    if (L->group) decode_down_kernel<true><<<grid, NTHREADS, SmemLayout::total, st>>>(a, R);
    else decode_down_kernel<false><<<grid, NTHREADS, SmemLayout::total, st>>>(a, R);
    count_launches(3);
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return fail(HMOE_E_CUDA, cudaGetErrorString(err));
    return HMOE_OK;
}

}  // namespace hmoe

// Router of the MoE layer: logits = x . Wt^T, sigmoid, + per-expert bias, top-k, renormalised fp16 weights.
// Replaces router_k (runtime/core/exl3_router.py:21-131) for any number of rows. Unlike the reference kernel (split-K
// with fp32 atomics, fast-math exp) every logit is summed in one fixed order with correctly rounded operations, and the
// sigmoid uses a fixed polynomial exp, so the selected experts are reproducible bit for bit by the CPU checker.
//   logit[r][e]: lane L of a warp sums columns i*256 + L*8 + j (i outer, j inner) with fused multiply-adds, then five
//   butterfly steps (xor 16, 8, 4, 2, 1) add the 32 partial sums.
// One launch: the block that completes a group of four rows last also selects their experts. Router calls that overlap
// on one device take different counter sets in rotation (sixteen of them).
#include <atomic>
#include "hmoe_common.cuh"
#include "hmoe_internal.h"
#include "hmoe_prepare.cuh"

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

constexpr int CTR_SLOTS = 16, CTR_GROUPS = 256;
// Arrival counters of the row groups, one set per call slot (calls take slots in rotation, so that calls overlapping on
// one device do not share counters unless more than CTR_SLOTS of them are in flight). Zero when the library is loaded;
// the block that arrives last puts its counter back to zero.
static __device__ unsigned g_router_ctr[CTR_SLOTS][CTR_GROUPS];
// Set by a block of the row group whose bounded wait gave up; read and cleared by the group's last block.
static __device__ unsigned g_router_bad[CTR_SLOTS][CTR_GROUPS];
// PREP: one count over all blocks of the launch in g_router_ctr[slot][0] (low half: arrivals, high half: blocks whose wait gave up).

// These kernels run once per layer on a handful of warps per SM: their duration is a chain of memory latencies, so every
// group of loads is issued before its first use.

// One warp selects NR rows (r, r + rstep, ...) of E <= 256 experts side by side: top-k rounds (max key, then lowest index holding
// it), weights. fresh: the logits were written by other blocks of the same launch (read them past L1). The rows' rounds are
// independent chains of warp-wide reductions, so two rows take little longer than one.
// Lane L keeps experts L, L + 32, ... (eight of them) of every row in registers: activation and order-preserving key. A round is
// seven compares per lane, one warp-wide maximum of the keys and one warp-wide minimum of the indices holding it; the winner's
// activation is broadcast from its lane and its key cleared there.
template <int NR>
__device__ __forceinline__ void topk_rows(const float* __restrict__ logits, const float* __restrict__ bias, int r, int rstep, int R, int E, int topk,
                                          float scale, int64_t* __restrict__ sel, __half* __restrict__ rw, int lane, bool fresh,
                                          int* s_sel_out = nullptr, float* s_rw_out = nullptr)
{
    float act[NR][8]; unsigned key[NR][8];
    {
        // all of the rows' logits and biases are requested before the first is used
        float l[NR][8], bb[8];
        #pragma unroll
        for (int i = 0; i < 8; ++i)
        {
            const int e = lane + 32 * i;
            #pragma unroll
            for (int n = 0; n < NR; ++n)
            {
                const int rr = r + n * rstep;
                l[n][i] = (e < E && rr < R) ? (fresh ? __ldcg(logits + (size_t) rr * E + e) : logits[(size_t) rr * E + e]) : 0.f;
            }
            bb[i] = (e < E && bias) ? __ldg(bias + e) : 0.f;
        }
        #pragma unroll
        for (int n = 0; n < NR; ++n)
            #pragma unroll
            for (int i = 0; i < 8; ++i)
            {
                act[n][i] = __fdiv_rn(1.f, __fadd_rn(1.f, det_expf(-l[n][i])));
                const unsigned u = __float_as_uint(__fadd_rn(act[n][i], bb[i]));
                key[n][i] = lane + 32 * i < E ? ((u & 0x80000000u) ? ~u : (u | 0x80000000u)) : 0u;
            }
    }
    float sum[NR], mine_w[NR]; int mine_id[NR];
    #pragma unroll
    for (int n = 0; n < NR; ++n) { sum[n] = 0.f; mine_w[n] = 0.f; mine_id[n] = 0; }
    #pragma unroll 1
    for (int k = 0; k < topk; ++k)
    {
        #pragma unroll
        for (int n = 0; n < NR; ++n)
        {
            unsigned lk = 0u; int li = lane;
            #pragma unroll
            for (int i = 0; i < 8; ++i) if (key[n][i] > lk) { lk = key[n][i]; li = lane + 32 * i; }     // ascending index: the lowest index wins a tie
            const unsigned m = __reduce_max_sync(0xffffffffu, lk);
            const unsigned bi = __reduce_min_sync(0xffffffffu, lk == m ? (unsigned) li : 0xffffffffu);
            float a = 0.f;
            #pragma unroll
            for (int i = 0; i < 8; ++i) if ((int) (bi >> 5) == i) a = act[n][i];
            a = __shfl_sync(0xffffffffu, a, (int) (bi & 31u));
            #pragma unroll
            for (int i = 0; i < 8; ++i) if ((int) bi == lane + 32 * i) key[n][i] = 0u;
            sum[n] = __fadd_rn(sum[n], a);
            if (lane == k) { mine_w[n] = a; mine_id[n] = (int) bi; }
        }
    }
    #pragma unroll
    for (int n = 0; n < NR; ++n)
    {
        const int rr = r + n * rstep;
        if (lane < topk && rr < R)
        {
            const __half h = __float2half_rn(__fdiv_rn(__fmul_rn(mine_w[n], scale), __fadd_rn(sum[n], 1e-20f)));
            sel[(size_t) rr * topk + lane] = mine_id[n];
            rw[(size_t) rr * topk + lane] = h;
            if (s_sel_out) { s_sel_out[rr * topk + lane] = mine_id[n]; s_rw_out[rr * topk + lane] = __half2float(h); }     // for a work list built by the same block
        }
    }
}
__device__ __noinline__ void topk_row(const float* __restrict__ logits, const float* __restrict__ bias, int r, int E, int topk, float scale,
                                      int64_t* __restrict__ sel, __half* __restrict__ rw, int lane, bool fresh, float* scratch)
{
    (void) scratch;
    topk_rows<1>(logits, bias, r, 0, r + 1, E, topk, scale, sel, rw, lane, fresh);
}

// Block (bx, by): experts 8 bx .. 8 bx + 7 (one per warp) x rows 4 by .. 4 by + 3, the columns in chunks of at most HC.
// Lane 0 of every warp brings the chunk of its expert's weight row into shared memory with one bulk copy, so all of a
// chunk's bytes are requested at once; meanwhile the block stages its rows as fp32 (two 16-byte halves per lane and step,
// halves of all lanes side by side: conflict-free). The sums then run from shared memory in the fixed order.
// With FUSED, the block that finishes a row group last (counted in g_router_ctr) also selects the group's experts.
constexpr int HC = 6144;

// NORM (the norm + router fusion, one chunk only): the rows come as the fp32 residual r (+ y); the block computes
// r' = r + y, the sum of squares of every row in the order of the stand-alone norm kernel (1024 virtual threads, float4
// columns t and t + 1024, butterflies), xn = fp16(r' * (w + cbias) * rsqrt(mean + eps) * cscale), and routes on xn, which is
// what a norm kernel followed by the router would do bit for bit. Blocks bx == 0 write r' and xn.
struct NormArgs
{
    const float* r; const float* y; float* r_out; const uint16_t* nw; __half* xn; float eps, cbias, cscale; int nw_bf16;
};

// PREP (with FUSED, without NORM): the launch also does the set-up step of the decode call that follows (hmoe_prepare.cuh), so that
// no separate prepare kernel sits between the router and the expert kernels: one more block per row group (blockIdx.x ==
// gridDim.x - 1) rewrites the group's rows for the MMAs while the other blocks compute logits, and the block that finishes last in
// the whole launch selects the experts of all rows and builds the Route.
// DISP (with PREP): expert parallelism with data-parallel tokens. The launch is also the dispatch: blocks (p, 0) for p < world first
// store this rank's rows into rank p's staging area and raise this rank's flag there (release, system scope); every block then
// waits, bounded, for the flags of the ranks that own its four rows before it reads them from the local staging area. So the
// exchange costs one NVLink round trip at the head of the router instead of a kernel of its own, and every rank routes all rows
// (the router is latency-bound: four rows or sixteen cost the same).
template <bool XBF, bool WBF, bool FUSED, bool NORM, bool PREP = false, bool DISP = false>
__global__ void __launch_bounds__(RW * 32) router_logits_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ wt,
                                                                int R, int H, int E, float* __restrict__ logits,
                                                                const float* __restrict__ bias, int topk, float scale,
                                                                int64_t* __restrict__ sel, __half* __restrict__ rw, int slot, const NormArgs na,
                                                                unsigned* __restrict__ status, const PrepArgs pa, const DispArgs da)
{
    extern __shared__ __align__(128) unsigned char rsm[];
    __shared__ int s_last;
    __shared__ int s_abort;
    __shared__ int s_blockbad;
    __shared__ __align__(8) unsigned long long s_bar[RW];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    TL_MIN(0);
    // The expert kernels that follow are launched with programmatic stream serialization: let their blocks be scheduled as this
    // kernel's blocks leave (they wait for this grid's completion before they read anything it wrote), so that their launch
    // latency and prologue overlap the selection in this kernel's last block.
    if (PREP) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int nrouter = PREP ? (int) gridDim.x - 1 : (int) gridDim.x;       // blocks per row group that compute logits
    if (PREP)
    {
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");    // the expert kernels' blocks may set up while this one runs
    }
    unsigned dgen = 0;                                   // DISP: this step's dispatch generation
    bool rows_ok = true;
    if (DISP)
    {
        __shared__ int s_rows_ok;
        unsigned* ctl = (unsigned*) (da.stage[da.rank] + da.ctl_off);      // [0] generation of the last step, [1] blocks of this launch that have read it
        dgen = *(volatile unsigned*) ctl + 1u;
        if (threadIdx.x == 0) s_rows_ok = 1;
        __syncthreads();
        if (threadIdx.x == 0) atomicAdd(ctl + 1, 1u);
        if (blockIdx.y == 0 && (int) blockIdx.x < da.world)
        {
            char* dst = da.stage[blockIdx.x];
            const int total = da.n_own * da.words;
            constexpr int U = 8;                            // all of a thread's loads are issued before its first store
            for (int base = threadIdx.x; base < total; base += RW * 32 * U)
            {
                uint4 v[U];
                #pragma unroll
                for (int u = 0; u < U; ++u) { const int i = base + u * RW * 32; if (i < total) v[u] = da.x_own[i]; }
                #pragma unroll
                for (int u = 0; u < U; ++u)
                {
                    const int i = base + u * RW * 32;
                    if (i < total) { const int j = i / da.words, c = i - j * da.words; ((uint4*) (dst + da.x_off))[(size_t) (da.rank + j * da.world) * da.words + c] = v[u]; }
                }
            }
            __syncthreads();
            if (threadIdx.x == 0) { __threadfence_system(); sys_st_release((unsigned*) (dst + da.flags_off) + da.rank, dgen); }
            TL_MAX(13);
        }
        if ((int) threadIdx.x < RR && (int) (blockIdx.y * RR + threadIdx.x) < R)
        {
            const unsigned* fl = (const unsigned*) (da.stage[da.rank] + da.flags_off) + (blockIdx.y * RR + threadIdx.x) % da.world;
            const unsigned long long t0 = globaltimer_ns();
            while ((int) (sys_ld_acquire(fl) - dgen) < 0)
                if (globaltimer_ns() - t0 > 2000000000ull) { atomicOr(pa.status, ST_WAIT_TIMEOUT); s_rows_ok = 0; break; }
        }
        __syncthreads();
        TL_MAX(15);
        rows_ok = s_rows_ok != 0;
    }
    if (PREP && (int) blockIdx.x == nrouter)
    {
        if (rows_ok)
            for (int r = blockIdx.y * RR; r < R && r < (int) (blockIdx.y + 1) * RR; ++r)
                prepare_row<DISP>(pa.x, pa.x_kind, r, H, pa.act_quant, pa.xf, pa.xscale, pa.gzero, pa.gzero_n, threadIdx.x, RW * 32);
        return;
    }
    const int hc = H < HC ? H : HC;                              // chunk length, a multiple of 256
    float* xs = (float*) rsm;                                    // [RR][hc] fp32, see above
    const uint32_t wsm = smem_u32(rsm) + RR * hc * 4 + warp * hc * 2, bar = smem_u32(&s_bar[warp]);
    const int r0 = blockIdx.y * RR, nr = R - r0 < RR ? R - r0 : RR;
    const int e = blockIdx.x * RW + warp;
    const uint16_t* w = wt + (size_t) (e < E ? e : 0) * H;
    if (lane == 0) { mbar_init(bar, 1); fence_barrier_init(); }
    if (threadIdx.x == 0) { s_abort = 0; s_blockbad = 0; }
    __syncthreads();
    float acc[RR];
    #pragma unroll
    for (int r = 0; r < RR; ++r) acc[r] = 0.f;
    uint32_t par = 0;
    #pragma unroll 1
    for (int c0 = 0; c0 < H; c0 += hc, par ^= 1)
    {
        const int cl = H - c0 < hc ? H - c0 : hc;
        if (c0 > 0) __syncthreads();                             // everyone is done with the previous chunk
        if (lane == 0) { mbar_expect_tx(bar, cl * 2); bulk_g2s(wsm, w + c0, cl * 2, bar); }
        if (NORM)
        {
            __shared__ float vsums[32];
            const int cols = H / 4, t = threadIdx.x;
            #pragma unroll 1
            for (int rr = 0; rr < RR; ++rr)
            {
                float4 v[4][2];                                   // virtual thread t + 256 k, float4 columns vt and vt + 1024
                float ps[4];
                #pragma unroll
                for (int k = 0; k < 4; ++k)
                    #pragma unroll
                    for (int j = 0; j < 2; ++j)
                    {
                        const int c = t + 256 * k + 1024 * j;
                        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (rr < nr && c < cols)
                        {
                            const size_t i = (size_t) (r0 + rr) * H + 4 * (size_t) c;
                            a = *(const float4*) (na.r + i);
                            if (na.y) { const float4 b = *(const float4*) (na.y + i); a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w; }
                        }
                        v[k][j] = a;
                    }
                #pragma unroll
                for (int k = 0; k < 4; ++k)
                {
                    // virtual thread t + 256 k of the stand-alone norm kernel: its two columns in order, then its warp's butterfly
                    float sq = 0.f;
                    #pragma unroll
                    for (int j = 0; j < 2; ++j)
                        if (t + 256 * k + 1024 * j < cols) sq = sq_accumulate(sq, v[k][j]);
                    ps[k] = butterfly32(sq);
                }
                __syncthreads();                                  // vsums free (previous row read)
                if (lane == 0) { vsums[warp] = ps[0]; vsums[warp + 8] = ps[1]; vsums[warp + 16] = ps[2]; vsums[warp + 24] = ps[3]; }
                __syncthreads();
                const float rmf = rsqrtf(butterfly32(vsums[lane]) / (float) H + na.eps) * na.cscale;
                #pragma unroll
                for (int k = 0; k < 4; ++k)
                    #pragma unroll
                    for (int j = 0; j < 2; ++j)
                    {
                        const int c = t + 256 * k + 1024 * j;
                        if (c >= cols) continue;
                        const float4 w4 = na.nw_bf16 ? norm_weight4<true>(na.nw, c) : norm_weight4<false>(na.nw, c);
                        const uint2 o = norm_pack4(v[k][j], w4, na.cbias, rmf);
                        // the router sees the rounded fp16 values, staged as fp32 in the order the logit sums read them
                        const float2 f0 = __half22float2(*(const __half2*) &o.x), f1 = __half22float2(*(const __half2*) &o.y);
                        const int col = 4 * c;
                        *(float4*) (xs + rr * hc + (col & ~255) + ((col & 255) >> 3) * 4 + (c & 1) * 128) = make_float4(f0.x, f0.y, f1.x, f1.y);
                        if (blockIdx.x == 0 && rr < nr)
                        {
                            const size_t i = (size_t) (r0 + rr) * H + col;
                            *(uint2*) (na.xn + i) = o;
                            if (na.r_out) *(float4*) (na.r_out + i) = v[k][j];
                        }
                    }
            }
        }
        else
        #pragma unroll 1
        for (int i0 = threadIdx.x * 8; i0 < RR * cl; i0 += RW * 32 * 8 * 6)
        {
            uint4 v[6];                                          // six loads in flight per thread
            #pragma unroll
            for (int u = 0; u < 6; ++u)
            {
                const int i = i0 + u * RW * 32 * 8, r = i / cl, c = i - r * cl;
                v[u] = (i < RR * cl && r < nr) ? (DISP ? __ldcg((const uint4*) (x + (size_t) (r0 + r) * H + c0 + c)) : *(const uint4*) (x + (size_t) (r0 + r) * H + c0 + c))
                                               : make_uint4(0, 0, 0, 0);
            }
            #pragma unroll
            for (int u = 0; u < 6; ++u)
            {
                const int i = i0 + u * RW * 32 * 8, r = i / cl, c = i - r * cl;
                if (i < RR * cl)
                {
                    float f[8];
                    widen8<XBF>(v[u], f);
                    float* d = xs + r * hc + (c & ~255) + ((c & 255) >> 3) * 4;
                    *(float4*) d = make_float4(f[0], f[1], f[2], f[3]);
                    *(float4*) (d + 128) = make_float4(f[4], f[5], f[6], f[7]);
                }
            }
        }
        __syncthreads();
        // A wait that gives up raises the status bit; the block skips the sums but still takes part in the arrival count
        // below, so the call's counter slot returns to zero and later calls that reuse it are not affected.
        const bool got = mbar_wait(bar, par, &s_abort, status) && rows_ok;
        if (FUSED && !got && lane == 0) { if (PREP) atomicOr(&s_blockbad, 1); else atomicOr(&g_router_bad[slot][blockIdx.y], 1u); }
        #pragma unroll 2
        for (int k = 0; got && k < cl; k += 256)
        {
            float wf[8];
            widen8<WBF>(lds128(wsm + (k + lane * 8) * 2), wf);
            const float* xk = xs + k + lane * 4;
            #pragma unroll
            for (int r = 0; r < RR; ++r)
            {
                const float4 a = *(const float4*) (xk + r * hc), b = *(const float4*) (xk + r * hc + 128);
                acc[r] = __fmaf_rn(a.x, wf[0], acc[r]); acc[r] = __fmaf_rn(a.y, wf[1], acc[r]);
                acc[r] = __fmaf_rn(a.z, wf[2], acc[r]); acc[r] = __fmaf_rn(a.w, wf[3], acc[r]);
                acc[r] = __fmaf_rn(b.x, wf[4], acc[r]); acc[r] = __fmaf_rn(b.y, wf[5], acc[r]);
                acc[r] = __fmaf_rn(b.z, wf[6], acc[r]); acc[r] = __fmaf_rn(b.w, wf[7], acc[r]);
            }
        }
    }
    #pragma unroll
    for (int r = 0; r < RR; ++r)
    {
        float a = acc[r];
        #pragma unroll
        for (int o = 16; o; o >>= 1) a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, o));
        if (lane == 0 && r < nr && e < E) logits[(size_t) (r0 + r) * E + e] = a;
    }
    if (!FUSED) return;
    TL_MAX(1);
    __threadfence();
    __syncthreads();
    if (PREP)
    {
        // One level: the block that finishes LAST IN THE WHOLE LAUNCH selects the experts of all rows (two rows per warp at sixteen
        // rows) and builds the work list from its own shared memory. Every hand-off through global memory costs about a
        // microsecond of latency on this chain (measured: logits 6.7 us after the kernel's entry, work list 17.5 us with the
        // group-wise scheme of the stand-alone router: an arrival count per row group, then one over the groups, each followed by a
        // flag load and a reload of what the previous step had written); here it is one arrival count, whose upper half carries
        // the "a wait gave up" flags, and one load of the logits.
        __shared__ unsigned s_old;
        if (threadIdx.x == 0)
        {
            unsigned* c = &g_router_ctr[slot][0];
            const unsigned old = atomicAdd(c, 1u + (s_blockbad ? 0x10000u : 0u));
            s_last = (old & 0xffffu) == (unsigned) nrouter * gridDim.y - 1u;
            s_old = old + (s_blockbad ? 0x10000u : 0u);
            if (s_last) *c = 0u;
        }
        __syncthreads();
        if (!s_last) return;
        __threadfence();
        const bool anybad = (s_old >> 16) != 0u;
        RouteSmem& S = *(RouteSmem*) (rsm + RW * 512 * 4);
        if (anybad)
        {
            // a wait gave up somewhere in this call: the logits are incomplete. Leave an empty Route (the expert kernels then do
            // nothing) and tell the host through the decode workspace's status word.
            if (threadIdx.x == 0) { atomicOr(pa.status, ST_WAIT_TIMEOUT); pa.route->m = 0; pa.route->ntiles = 0; }
            for (int i = threadIdx.x; i < 2 * (MAXB + 1); i += RW * 32) pa.route->split[i / (MAXB + 1)][i % (MAXB + 1)] = 0;
        }
        else
        {
            // R <= 16: rows warp and warp + 8 (one instance of the code whatever R is: this block runs it once, from a cold instruction cache)
            if (warp < R) topk_rows<2>(logits, bias, warp, RW, R, E, topk, scale, sel, rw, lane, true, S.raw_sel, S.s_rw);
        }
        TL_MAX(3);
        if (DISP && threadIdx.x == 0)
        {
            // this block is the last to work: once every block of the launch has read the generation, advance it (bounded wait)
            unsigned* ctl = (unsigned*) (da.stage[da.rank] + da.ctl_off);
            const unsigned nblk = gridDim.x * gridDim.y;
            const unsigned long long t0 = globaltimer_ns();
            while (*(volatile unsigned*) (ctl + 1) < nblk)
                if (globaltimer_ns() - t0 > 1000000000ull) { atomicOr(pa.status, ST_WAIT_TIMEOUT); break; }
            ctl[1] = 0u;
            *(volatile unsigned*) ctl = dgen;
        }
        __syncthreads();
        if (anybad) return;
        build_route<2>(S, sel, rw, R, H, pa.I, topk, pa.lo, pa.n_local, pa.has_shared, pa.sh_mod, pa.sh_rem,
                       pa.gen_bump, pa.route, pa.nblocks, threadIdx.x, pa.n_total, pa.bal_world, pa.bal_rank);
        TL_MAX(5);
        return;
    }
    if (threadIdx.x == 0)
    {
        unsigned* c = &g_router_ctr[slot][blockIdx.y];
        const unsigned old = atomicAdd(c, 1u);
        s_last = old == (unsigned) nrouter - 1;
        if (s_last) *c = 0u;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    {
        // after a failed wait the logits are incomplete: select nothing (the status word tells the host)
        const unsigned bad = *(volatile unsigned*) &g_router_bad[slot][blockIdx.y];
        __syncthreads();
        if (threadIdx.x == 0 && bad) g_router_bad[slot][blockIdx.y] = 0u;
        if (bad) return;
        if (warp < nr) topk_row(logits, bias, r0 + warp, E, topk, scale, sel, rw, lane, true, xs + warp * 512);
    }
}

__global__ void __launch_bounds__(256) router_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int R, int E,
                                                         int topk, float scale, int64_t* __restrict__ sel, __half* __restrict__ rw)
{
    __shared__ float scratch[8 * 512];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, r = blockIdx.x * 8 + warp;
    if (r < R) topk_row(logits, bias, r, E, topk, scale, sel, rw, lane, false, scratch + warp * 512);
}

template <bool XBF, bool WBF>
void launch_logits(dim3 grid, size_t smem, cudaStream_t st, bool fused, const uint16_t* x, const uint16_t* wt, int R, int H, int E,
                   float* logits, const float* bias, int topk, float scale, int64_t* sel, __half* rw, int slot, unsigned* status)
{
    static DeviceOnce once;
    if (once.first())
    {
        cudaFuncSetAttribute(router_logits_kernel<XBF, WBF, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(router_logits_kernel<XBF, WBF, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    }
    const NormArgs na = {};
    if (fused) router_logits_kernel<XBF, WBF, true, false><<<grid, RW * 32, smem, st>>>(x, wt, R, H, E, logits, bias, topk, scale, sel, rw, slot, na, status, PrepArgs(), DispArgs());
    else router_logits_kernel<XBF, WBF, false, false><<<grid, RW * 32, smem, st>>>(x, wt, R, H, E, logits, bias, topk, scale, sel, rw, slot, na, status, PrepArgs(), DispArgs());
}

template <bool WBF>
void launch_norm_router(dim3 grid, size_t smem, cudaStream_t st, bool fused, const uint16_t* wt, int R, int H, int E, float* logits,
                        const float* bias, int topk, float scale, int64_t* sel, __half* rw, int slot, const NormArgs& na, unsigned* status)
{
    static DeviceOnce once;
    if (once.first())
    {
        cudaFuncSetAttribute(router_logits_kernel<false, WBF, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(router_logits_kernel<false, WBF, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    }
    if (fused) router_logits_kernel<false, WBF, true, true><<<grid, RW * 32, smem, st>>>(nullptr, wt, R, H, E, logits, bias, topk, scale, sel, rw, slot, na, status, PrepArgs(), DispArgs());
    else router_logits_kernel<false, WBF, false, true><<<grid, RW * 32, smem, st>>>(nullptr, wt, R, H, E, logits, bias, topk, scale, sel, rw, slot, na, status, PrepArgs(), DispArgs());
}

// Both entry points share the counter sets, so they also share the rotation that hands them out.
std::atomic<unsigned> g_router_calls{0};

template <bool XBF, bool WBF>
void launch_logits_prep(dim3 grid, size_t smem, cudaStream_t st, const uint16_t* x, const uint16_t* wt, int R, int H, int E, float* logits,
                        const float* bias, int topk, float scale, int64_t* sel, __half* rw, int slot, unsigned* status, const PrepArgs& pa,
                        const DispArgs* da)
{
    static DeviceOnce once;
    if (once.first())
    {
        cudaFuncSetAttribute(router_logits_kernel<XBF, WBF, true, false, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(router_logits_kernel<XBF, WBF, true, false, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    }
    const NormArgs na = {};
    if (da) router_logits_kernel<XBF, WBF, true, false, true, true><<<grid, RW * 32, smem, st>>>(x, wt, R, H, E, logits, bias, topk, scale, sel, rw, slot, na, status, pa, *da);
    else router_logits_kernel<XBF, WBF, true, false, true, false><<<grid, RW * 32, smem, st>>>(x, wt, R, H, E, logits, bias, topk, scale, sel, rw, slot, na, status, pa, DispArgs());
}

}  // namespace

// workspace: status word (256 bytes, see hmoe_ws_status) + logits fp32 [R][E]
size_t router_ws_bytes(int R, int E) { return 256 + ((size_t) R * E * 4 + 255) / 256 * 256; }

int router_launch(const void* x, int x_dtype, const void* wt, int w_dtype, const float* bias, int R, int H, int E, int topk,
                  float scale, int64_t* sel, void* rw, void* ws, size_t ws_bytes, cudaStream_t st)
{
    if (R < 1 || E < 32 || E > 256 || E % 32 || H % 256 || H < 256 || topk < 1 || topk > TOPK_MAX || topk > E)
        return fail(HMOE_E_ARG, "hmoe_router: needs R >= 1, E % 32 == 0, E <= 256, H % 256 == 0, topk <= 8");
    if ((x_dtype != HMOE_F16 && x_dtype != HMOE_BF16) || (w_dtype != HMOE_F16 && w_dtype != HMOE_BF16))
        return fail(HMOE_E_ARG, "hmoe_router: x and wt must be fp16 or bf16");
    if (!x || !wt || !sel || !rw || !ws) return fail(HMOE_E_ARG, "hmoe_router: null pointer");
    if (ws_bytes < router_ws_bytes(R, E)) return fail(HMOE_E_WS, "hmoe_router: workspace too small");
    const int hc = H < HC ? H : HC;
    const size_t smem = (size_t) RR * (hc > 512 ? hc : 512) * 4 + (size_t) RW * hc * 2;    // rows as fp32 (reused as the selection's scratch) + weight rows
    const dim3 grid((E + RW - 1) / RW, (R + RR - 1) / RR);
    unsigned* status = (unsigned*) ws;
    float* logits = (float*) ((char*) ws + 256);
    const uint16_t* xp = (const uint16_t*) x; const uint16_t* wp = (const uint16_t*) wt;
    // Up to CTR_GROUPS row groups the selection runs in the same launch (the last block of a row group does it); beyond,
    // a second kernel selects.
    const bool fused = (int) grid.y <= CTR_GROUPS;
    const int slot = (int) (g_router_calls.fetch_add(1, std::memory_order_relaxed) % CTR_SLOTS);
    const bool xb = x_dtype == HMOE_BF16, wb = w_dtype == HMOE_BF16;
    if (!xb && !wb) launch_logits<false, false>(grid, smem, st, fused, xp, wp, R, H, E, logits, bias, topk, scale, sel, (__half*) rw, slot, status);
    else if (!xb && wb) launch_logits<false, true>(grid, smem, st, fused, xp, wp, R, H, E, logits, bias, topk, scale, sel, (__half*) rw, slot, status);
    else if (xb && !wb) launch_logits<true, false>(grid, smem, st, fused, xp, wp, R, H, E, logits, bias, topk, scale, sel, (__half*) rw, slot, status);
    else launch_logits<true, true>(grid, smem, st, fused, xp, wp, R, H, E, logits, bias, topk, scale, sel, (__half*) rw, slot, status);
    if (!fused) router_topk_kernel<<<(R + 7) / 8, 256, 0, st>>>(logits, bias, R, E, topk, scale, sel, (__half*) rw);
    count_launches(fused ? 1 : 2);
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return fail(HMOE_E_CUDA, cudaGetErrorString(err));
    return HMOE_OK;
}

// The router with the decode call's set-up step inside its launch: `pa` comes from decode_prep_args.
int router_prepare_launch(const void* x, int x_dtype, const void* wt, int w_dtype, const float* bias, int R, int H, int E, int topk, float scale,
                          int64_t* sel, void* rw, void* ws, size_t ws_bytes, const PrepArgs& pa, cudaStream_t st, const DispArgs* da)
{
    if (R < 1 || R > MAXR || E < 32 || E > 256 || E % 32 || H % 256 || H < 256 || topk < 1 || topk > TOPK_MAX || topk > E)
        return fail(HMOE_E_ARG, "hmoe_router_decode: needs 1 <= R <= 16, E % 32 == 0, E <= 256, H % 256 == 0, topk <= 8");
    if ((x_dtype != HMOE_F16 && x_dtype != HMOE_BF16) || (w_dtype != HMOE_F16 && w_dtype != HMOE_BF16))
        return fail(HMOE_E_ARG, "hmoe_router_decode: x and wt must be fp16 or bf16");
    if (!x || !wt || !sel || !rw || !ws) return fail(HMOE_E_ARG, "hmoe_router_decode: null pointer");
    if (ws_bytes < router_ws_bytes(R, E)) return fail(HMOE_E_WS, "hmoe_router_decode: router workspace too small");
    const int hc = H < HC ? H : HC;
    size_t smem = (size_t) RR * (hc > 512 ? hc : 512) * 4 + (size_t) RW * hc * 2;
    const size_t need = (size_t) RW * 512 * 4 + sizeof(RouteSmem);            // the selection's scratch, then the Route builder's
    if (smem < need) smem = need;
    const dim3 grid((E + RW - 1) / RW + 1, (R + RR - 1) / RR);                // + 1: the block that rewrites the group's rows
    unsigned* status = (unsigned*) ws;
    float* logits = (float*) ((char*) ws + 256);
    const uint16_t* xp = (const uint16_t*) x; const uint16_t* wp = (const uint16_t*) wt;
    const int slot = (int) (g_router_calls.fetch_add(1, std::memory_order_relaxed) % CTR_SLOTS);
    const bool xb = x_dtype == HMOE_BF16, wb = w_dtype == HMOE_BF16;
    if (!xb && !wb) launch_logits_prep<false, false>(grid, smem, st, xp, wp, R, H, E, logits, bias, topk, scale, sel, (__half*) rw, slot, status, pa, da);
    else if (!xb && wb) launch_logits_prep<false, true>(grid, smem, st, xp, wp, R, H, E, logits, bias, topk, scale, sel, (__half*) rw, slot, status, pa, da);
    else if (xb && !wb) launch_logits_prep<true, false>(grid, smem, st, xp, wp, R, H, E, logits, bias, topk, scale, sel, (__half*) rw, slot, status, pa, da);
    else launch_logits_prep<true, true>(grid, smem, st, xp, wp, R, H, E, logits, bias, topk, scale, sel, (__half*) rw, slot, status, pa, da);
    count_launches(1);
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return fail(HMOE_E_CUDA, cudaGetErrorString(err));
    return HMOE_OK;
}

int norm_router_launch(const float* y, const float* r, float* r_out, const void* nw, int nw_dtype, void* xn, const void* wt, int w_dtype,
                       const float* bias, int R, int H, int E, int topk, float scale, float eps, float cbias, float cscale, int64_t* sel, void* rw,
                       void* ws, size_t ws_bytes, cudaStream_t st)
{
    if (R < 1 || E < 32 || E > 256 || E % 32 || H % 256 || H < 256 || H > HC || topk < 1 || topk > TOPK_MAX || topk > E)
        return fail(HMOE_E_ARG, "hmoe_norm_router: needs R >= 1, E % 32 == 0, E <= 256, H % 256 == 0, H <= 6144, topk <= 8");
    if ((nw_dtype != HMOE_F16 && nw_dtype != HMOE_BF16) || (w_dtype != HMOE_F16 && w_dtype != HMOE_BF16))
        return fail(HMOE_E_ARG, "hmoe_norm_router: the norm weight and wt must be fp16 or bf16");
    if (!r || !nw || !xn || !wt || !sel || !rw || !ws || r_out == r || (y && r_out == y)) return fail(HMOE_E_ARG, "hmoe_norm_router: null pointer, or r_out aliases an input");
    if (ws_bytes < router_ws_bytes(R, E)) return fail(HMOE_E_WS, "hmoe_norm_router: workspace too small");
    const size_t smem = (size_t) RR * (H > 512 ? H : 512) * 4 + (size_t) RW * H * 2;
    const dim3 grid((E + RW - 1) / RW, (R + RR - 1) / RR);
    const bool fused = (int) grid.y <= CTR_GROUPS;
    const int slot = (int) (g_router_calls.fetch_add(1, std::memory_order_relaxed) % CTR_SLOTS);
    NormArgs na;
    na.r = r; na.y = y; na.r_out = r_out; na.nw = (const uint16_t*) nw; na.xn = (__half*) xn; na.eps = eps; na.cbias = cbias; na.cscale = cscale;
    na.nw_bf16 = nw_dtype == HMOE_BF16;
    unsigned* status = (unsigned*) ws;
    float* logits = (float*) ((char*) ws + 256);
    if (w_dtype == HMOE_BF16) launch_norm_router<true>(grid, smem, st, fused, (const uint16_t*) wt, R, H, E, logits, bias, topk, scale, sel, (__half*) rw, slot, na, status);
    else launch_norm_router<false>(grid, smem, st, fused, (const uint16_t*) wt, R, H, E, logits, bias, topk, scale, sel, (__half*) rw, slot, na, status);
    if (!fused) router_topk_kernel<<<(R + 7) / 8, 256, 0, st>>>(logits, bias, R, E, topk, scale, sel, (__half*) rw);
    count_launches(fused ? 1 : 2);
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return fail(HMOE_E_CUDA, cudaGetErrorString(err));
    return HMOE_OK;
}

}  // namespace hmoe

#ifdef HMOE_PROBE_TIMELINE
using namespace hmoe;
TL_READER(hmoe_tl_router)
#endif

// The set-up step of a decode call, as device functions, so that it can run as a kernel of its own (decode_prepare_kernel) or
// inside the router's launch (router_logits_kernel with its PREP option): one row's activations rewritten for the MMAs, and
// the Route built from the selection.
#pragma once
#include "hmoe_common.cuh"

namespace hmoe {

// Row r of x rewritten as fp16 in the column order the MMAs read (in the int8 mode: the CPU engine's int8 codes as fp16 integers
// plus a scale per 32 columns), and the row's share of the per-pick gate / up sums cleared. Called by `nthreads` threads of a block.
// FRESH: the row arrived from another GPU during this launch (read it past L1).
template <bool FRESH = false>
__device__ __forceinline__ void prepare_row(const void* __restrict__ x, int x_kind /* 0 fp16, 1 bf16, 2 fp16 in MMA column order */, int r, int H,
                                            int act_quant, __half* __restrict__ xf, float* __restrict__ xscale, float4* __restrict__ gzero,
                                            int gzero_n, int tid, int nthreads)
{
    // this row's share of the gate / up sums is cleared for the streaming kernels' reductions (gzero_n float4 per row block)
    for (int i = tid; i < gzero_n; i += nthreads) gzero[(size_t) r * gzero_n + i] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int gi = tid; gi < H / 32; gi += nthreads)
    {
        float v[32];
        if (x_kind == 2)
        {
            // fp16 rows that already are in the MMA column order (the copy the reference's norm + router kernel can write for
            // moe4, its xf argument): word p of the 64-column block sits at frag_pos(p)
            const uint32_t* src = (const uint32_t*) ((const uint16_t*) x + (size_t) r * H + (gi >> 1) * 64);
            #pragma unroll
            for (int p = 0; p < 16; ++p)
            {
                const uint32_t w = src[frag_pos((gi & 1) * 16 + p)];
                const float2 f = __half22float2(*(const __half2*) &w);
                v[2 * p] = f.x; v[2 * p + 1] = f.y;
            }
        }
        else
        {
            const uint4* p = (const uint4*) ((const uint16_t*) x + (size_t) r * H + gi * 32);
            #pragma unroll
            for (int j = 0; j < 4; ++j)
            {
                const uint4 u = FRESH ? __ldcg(p + j) : p[j];
                const uint32_t w[4] = {u.x, u.y, u.z, u.w};
                #pragma unroll
                for (int k = 0; k < 4; ++k)
                {
                    if (x_kind == 1) { v[j * 8 + 2 * k] = __uint_as_float(w[k] << 16); v[j * 8 + 2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u); }
                    else { const float2 f = __half22float2(*(const __half2*) &w[k]); v[j * 8 + 2 * k] = f.x; v[j * 8 + 2 * k + 1] = f.y; }
                }
            }
        }
        if (act_quant)
        {
            // the CPU engine's activation format (runtime/tier/cpuband.cpp:106-111): int8 with a scale per 32 values.
            // The codes themselves go to the MMAs (exact in fp16), the scale is applied to the fp32 sums.
            float m = 0.f;
            #pragma unroll
            for (int k = 0; k < 32; ++k) m = fmaxf(m, fabsf(v[k]));
            const float s = m > 0.f ? __fdiv_rn(m, 127.f) : 1.f;
            const float inv = __fdiv_rn(1.f, s);
            #pragma unroll
            for (int k = 0; k < 32; ++k) v[k] = (float) __float2int_rn(__fmul_rn(v[k], inv));
            xscale[(size_t) r * (H / 32) + gi] = s;
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
}

// What the set-up step needs beyond the routing itself, gathered by the host (decode_prep_args) so that the router's launch can
// do the step in place of decode_prepare_kernel.
struct PrepArgs
{
    int n_total = 0, bal_world = 0, bal_rank = 0;       // experts held by two ranks (see build_route); 0 = off
    const void* x; int x_kind, act_quant;
    __half* xf; float* xscale; float4* gzero; int gzero_n;
    Route* route;
    int lo, n_local, has_shared, sh_mod, sh_rem;
    unsigned* gen_bump;
    int I, nblocks;
    unsigned* status;          // the decode workspace's status word
};

// Expert parallelism with data-parallel tokens: what the router's launch needs to do the dispatch itself (push this rank's rows
// into every rank's staging area, wait for the rows of its row group). stage[p] = rank p's staging area as seen from here.
struct DispArgs
{
    int rank, world, n_own, words;      // rows this rank owns (rank, rank + world, ...), 16-byte words per row
    char* stage[8];
    const uint4* x_own;                 // [n_own][H] 2-byte elements
    size_t x_off, flags_off, ctl_off;   // StageLayout offsets
};

// Shared memory of build_route (17 KB).
struct RouteSmem
{
    short slot_of[256];                        // local expert id -> slot, -1 if not picked
    short slot_e[MAXS];
    unsigned s_mask[MAXS];                     // rows of the slot, one bit each
    unsigned char s_rows[MAXS][MAXR];
    float s_w[MAXS][MAXR];
    int s_scan[4][256];                        // per slot: tiles, rows, cost in gate_up, cost in down (then their prefix sums)
    int s_cum[2][MAXT + 1];
    short s_sel[MAXR * TOPK_MAX];
    float s_rw[MAXR * TOPK_MAX];
    int wcount[8];
    int m_sh;
    unsigned char gflag[256];                  // replicated experts: router position -> 1 picked by some row, 2 picked and served here
    int raw_sel[MAXR * TOPK_MAX];              // SRC = 2: the selections (router positions) and, in s_rw, the weights, left here by the
};                                             // block's own selection step instead of being read back from global memory

// routing block: slot = distinct expert (ascending id), then the shared expert; tiles of <= 8 rows per slot.
// Everything is done in parallel with block-wide prefix sums: this block is the critical path of the call (the
// streaming kernel's blocks are already resident and wait for it).
// Called by all 256 threads of one block. SRC = 1: sel / rw were written by other blocks of the same launch (read them past L1);
// SRC = 2: they are in S.raw_sel / S.s_rw already (written by this block's own selection step, visible after a barrier).
template <int SRC>
__device__ __forceinline__ void build_route(RouteSmem& S, const int64_t* __restrict__ sel, const __half* __restrict__ rw, int R, int H, int I, int topk,
                                            int lo, int n_local, int has_shared, int sh_mod, int sh_rem, unsigned* gen_bump,
                                            Route* __restrict__ route, int nblocks, int tid, int n_total = 0, int bal_world = 0, int bal_rank = 0)
{
    const int NP = R * topk;
    S.slot_of[tid] = 0;                                      // used as the picked flag first
    if (tid < MAXS) S.s_mask[tid] = 0u;
    if (bal_world <= 1) __syncthreads();                     // (the other path has its own barriers before the flags are set)
    if (bal_world > 1)
    {
        // Every expert held by two ranks (rank r holds the bands r and r + 1 of n_total / world positions each, so position e is
        // held by its band's rank p and by rank p - 1): which of the two serves a picked expert this step is decided here, by
        // every rank alike from the same selections. One warp, lane = band: the bands walk their positions side by side and
        // give each picked one to the holder with fewer experts so far (ties: the band's own rank). Measured over random
        // top-8 routings of 16 rows: most loaded rank 26.1 instead of 29.5 experts at 4 ranks, 13.8 instead of 16.7 at 8.
        S.gflag[tid] = 0;
        __syncthreads();
        if (tid < NP)
        {
            const int64_t e = SRC == 2 ? (int64_t) S.raw_sel[tid] : SRC == 1 ? (int64_t) __ldcg((const long long*) sel + tid) : sel[tid];
            if (e >= 0 && e < n_total) S.gflag[(int) e] = 1;
        }
        __syncthreads();
        if (tid < 32)
        {
            const int npr = n_total / bal_world, band = tid, prev = (tid + bal_world - 1) % bal_world;
            int load = 0;                                    // lane r: experts given to rank r so far
            for (int i = 0; i < npr; ++i)
            {
                const int load_prev = __shfl_sync(0xffffffffu, load, prev % 32);
                const bool picked = band < bal_world && S.gflag[band * npr + i] != 0;
                const bool to_prev = picked && load_prev < load;
                const unsigned own = __ballot_sync(0xffffffffu, picked && !to_prev), oth = __ballot_sync(0xffffffffu, to_prev);
                if (band < bal_world)
                {
                    load += (int) ((own >> band) & 1u) + (int) ((oth >> ((band + 1) % bal_world)) & 1u);
                    if (picked && (to_prev ? prev : band) == bal_rank) S.gflag[band * npr + i] = 2;
                }
            }
        }
        __syncthreads();
    }
    if (tid < NP)
    {
        int64_t e = SRC == 2 ? (int64_t) S.raw_sel[tid] : SRC == 1 ? (int64_t) __ldcg((const long long*) sel + tid) : sel[tid];
        bool in;
        if (bal_world > 1)
        {
            in = e >= 0 && e < n_total && S.gflag[(int) e] == 2;
            e -= lo;
            if (e < 0) e += n_total;                         // the second band of the last rank wraps around to position 0
        }
        else { e -= lo; in = e >= 0 && e < n_local; }
        S.s_sel[tid] = in ? (short) e : (short) -1;
        if (SRC != 2) S.s_rw[tid] = __half2float(SRC == 1 ? __ushort_as_half(__ldcg((const unsigned short*) rw + tid)) : rw[tid]);
        if (in) S.slot_of[(int) e] = 1;
    }
    __syncthreads();
    TL_MAX(7);
    {
        // distinct experts in ascending order: one flag per thread, ballots per warp, prefix over the eight warps
        const bool picked = S.slot_of[tid] != 0;
        const unsigned bl = __ballot_sync(0xffffffffu, picked);
        if ((tid & 31) == 0) S.wcount[tid >> 5] = __popc(bl);
        __syncthreads();
        int before = 0, m = 0;
        for (int w = 0; w < 8; ++w) { if (w < (tid >> 5)) before += S.wcount[w]; m += S.wcount[w]; }
        const int slot = before + __popc(bl & ((1u << (tid & 31)) - 1u));
        S.slot_of[tid] = picked ? (short) slot : (short) -1;
        if (picked) S.slot_e[slot] = (short) tid;
        if (tid == 0) { S.m_sh = m; if (has_shared) S.slot_e[m] = -1; }
    }
    __syncthreads();
    const int m = S.m_sh, ns = m + (has_shared ? 1 : 0);
    // one thread per pick: the first pick of an expert in its row owns the (slot, row) pair and the summed weight
    int my_slot = -1, my_row = 0; float my_w = 0.f;
    if (tid < NP && S.s_sel[tid] >= 0)
    {
        const int r = tid / topk, k = tid - r * topk, e = S.s_sel[tid];
        bool first = true;
        for (int k2 = 0; k2 < k; ++k2) first &= S.s_sel[r * topk + k2] != e;
        if (first)
        {
            for (int k2 = k; k2 < topk; ++k2) if (S.s_sel[r * topk + k2] == e) my_w += S.s_rw[r * topk + k2];
            my_slot = S.slot_of[e]; my_row = r;
            atomicOr(&S.s_mask[my_slot], 1u << r);
        }
    }
    // the shared expert takes every row with weight 1; under expert parallelism only rows r % sh_mod == sh_rem here
    if (has_shared && tid >= 128 && tid < 128 + R && (tid - 128) % sh_mod == sh_rem) atomicOr(&S.s_mask[m], 1u << (tid - 128));
    __syncthreads();
    if (my_slot >= 0)
    {
        const int pos = __popc(S.s_mask[my_slot] & ((1u << my_row) - 1u));
        S.s_rows[my_slot][pos] = (unsigned char) my_row; S.s_w[my_slot][pos] = my_w;
    }
    if (has_shared && tid >= 128 && tid < 128 + R && (tid - 128) % sh_mod == sh_rem)
    {
        const int pos = __popc(S.s_mask[m] & ((1u << (tid - 128)) - 1u));
        S.s_rows[m][pos] = (unsigned char) (tid - 128); S.s_w[m][pos] = 1.f;
    }
    // Per slot: tiles, rows, and the cost of its items in the two streaming kernels. The kernels are bound by HBM, but an
    // item of a tile with many real rows issues more reductions and runs a little longer (measured: 8 rows against 1,
    // +20 % in down, under +1 % in gate_up); the blocks' item ranges are cut at equal cost so that the blocks that get the
    // 16-row shared expert do not finish last.
    const int J0 = 2 * (I / 64), J1 = H / 64;
    TL_MAX(9);
    // inclusive prefix sums of the four columns over the 256 threads: shuffles inside the warps, the eight warp totals through
    // shared memory (two barriers)
    int incl[4];
    {
        const int n = tid < ns ? __popc(S.s_mask[tid]) : 0, full = n >> 3, rest = n & 7;
        incl[0] = (n + 7) >> 3;
        incl[1] = n;
        incl[2] = J0 * (full * (400 + 8) + (rest ? 400 + rest : 0));
        incl[3] = J1 * (full * (100 + 3 * 8) + (rest ? 100 + 3 * rest : 0));
    }
    const int lane_ = tid & 31, warp_ = tid >> 5;
    #pragma unroll
    for (int o = 1; o < 32; o <<= 1)
        #pragma unroll
        for (int c = 0; c < 4; ++c) { const int t = __shfl_up_sync(0xffffffffu, incl[c], o); if (lane_ >= o) incl[c] += t; }
    if (lane_ == 31)
        #pragma unroll
        for (int c = 0; c < 4; ++c) S.s_scan[c][warp_] = incl[c];
    __syncthreads();
    int tot[4];
    #pragma unroll
    for (int c = 0; c < 4; ++c)
    {
        int before = 0, all = 0;
        #pragma unroll
        for (int w = 0; w < 8; ++w) { const int x = S.s_scan[c][w]; all += x; if (w < warp_) before += x; }
        incl[c] += before; tot[c] = all;
    }
    __syncthreads();                                       // s_scan is reused below
    const int nt = tot[0];
    if (tid == 0)
    {
        route->m = m; route->ntiles = nt; route->pad[0] = route->pad[1] = 0;
        S.s_cum[0][nt] = tot[2]; S.s_cum[1][nt] = tot[3];
        if (gen_bump) *gen_bump += 1;          // expert-parallel step counter: selects the partial slot and the combine's generation
    }
    if (tid < ns)
    {
        const int n = __popc(S.s_mask[tid]);
        int t = incl[0] - ((n + 7) >> 3), rb = incl[1] - n;
        int c0 = incl[2] - J0 * ((n >> 3) * 408 + ((n & 7) ? 400 + (n & 7) : 0)), c1 = incl[3] - J1 * ((n >> 3) * 124 + ((n & 7) ? 100 + 3 * (n & 7) : 0));
        for (int b8 = 0; b8 < n; b8 += 8, ++t)
        {
            const int nn = n - b8 < 8 ? n - b8 : 8;
            route->expert[t] = S.slot_e[tid]; route->nrows[t] = (unsigned char) nn; route->rowbase[t] = (short) (rb + b8);
            for (int i = 0; i < 8; ++i)
            {
                route->rows[t][i] = S.s_rows[tid][b8 + (i < nn ? i : 0)];
                route->w[t][i] = i < nn ? S.s_w[tid][b8 + i] : 0.f;
            }
            S.s_cum[0][t] = c0; S.s_cum[1][t] = c1;
            S.s_scan[0][t] = nn;                 // rows of tile t (the tile counts are no longer needed: every thread holds its own)
            c0 += J0 * (400 + nn); c1 += J1 * (100 + 3 * nn);
        }
    }
    __syncthreads();
    TL_MAX(11);
    for (int i = tid; i < 2 * (nblocks + 1); i += 256)
    {
        const int k = i / (nblocks + 1), b = i % (nblocks + 1), J = k ? J1 : J0;
        int p = nt * J;
        if (b < nblocks && nt > 0)
        {
            const int target = (int) ((long long) S.s_cum[k][nt] * b / nblocks);
            int lo2 = 0, hi = nt - 1;                    // last tile whose start is <= target
            while (lo2 < hi) { const int mid = (lo2 + hi + 1) >> 1; if (S.s_cum[k][mid] <= target) lo2 = mid; else hi = mid - 1; }
            const int item = k ? 100 + 3 * S.s_scan[0][lo2] : 400 + S.s_scan[0][lo2];
            const int off = (target - S.s_cum[k][lo2]) / item;
            p = lo2 * J + (off < J ? off : J);
        }
        route->split[k][b] = p;
    }
}

}  // namespace hmoe

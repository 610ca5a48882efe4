// Decode path of the MoE expert layer (<= 16 rows: tokens and their MTP drafts), sm_100a.
//
// Replaces the reference's moe4 decode kernels (runtime/tier/moe4/moe4.cu:361-676: moe4_a_kernel, moe4_act_kernel,
// moe4_b_kernel and their in-kernel route()) behind the same operator surface: packed int4 experts in the reference's
// fragment order, routing as (sel, rw), fp32 output accumulated into y. Differences by design: 16 rows in one pass over
// the weights, a scale per 128 input columns (or the reference's scale per row), an int4 shared expert as one more expert.
//
// Launches per call:
//   prepare : one block per row rewrites x as fp16 in the column order the MMAs read (in the int8 mode: the CPU engine's
//             int8 codes as fp16 integers plus a scale per 32 columns) and clears the per-pick sums; one more block builds the
//             Route: the distinct experts, each with the <= 8 rows that picked it as one tile, and the item ranges of the
//             streaming kernels' blocks.
//   H <= 6144 and I <= 2048 (the register-resident path, see decode_stream_kernel):
//     gate_up, down : the same persistent streaming kernel, one block per SM, 16 warps with private rings of 1-D bulk
//             copies; gate and up sums go to a per-pick fp32 buffer, down turns them into its operand when it enters a tile.
//   larger shapes (decode_gate_up_kernel, decode_down_kernel): the tile's activation fragments no longer fit in registers
//             and are fetched stage by stage; gate_up reduces its sixteen partial tiles through shared memory and writes
//             act = SiLU(gate) * up * weight as fp16, down adds every tile's contribution to a 64-column slice of y in shared
//             memory.
//   The reference's int8 shared expert, when the layer has one, runs as two more small kernels (hmoe_shared_i8.cu).
// All streaming kernels are bound by HBM: algorithmic bytes per call are (distinct experts + shared) x the expert's
// packed size plus scales.
#include "hmoe_common.cuh"
#include "hmoe_internal.h"
#include "hmoe_prepare.cuh"

namespace hmoe {

namespace {

constexpr int CW = 16;                   // warps per block
constexpr int NTHREADS = CW * 32;
constexpr int STAGE_BYTES = 65536;       // 32 units of 64 rows x 64 columns
constexpr int NSTAGE = 3;
constexpr int NBUF = 4;                  // gate_up partial-sum buffers in rotation (a warp runs at most NSTAGE items ahead)
constexpr int GU_FLOATS = 2 * 64 * 8;    // [matrix][64 rows][8 tile columns]
constexpr int YACC_FLOATS = MAXR * 64;
constexpr int YCOPIES = 8;                // copies of the down kernel's output slice (two warps share one)

struct SmemLayout
{
    static constexpr int ring = 0;
    static constexpr int gu = NSTAGE * STAGE_BYTES;                   // gate_up: NBUF x GU_FLOATS; down: YACC_FLOATS
    static constexpr int bars = gu + (NBUF * GU_FLOATS > YCOPIES * YACC_FLOATS ? NBUF * GU_FLOATS : YCOPIES * YACC_FLOATS) * 4;   // full[NSTAGE][CW]
    static constexpr int cnt = bars + NSTAGE * CW * 8;                // NBUF arrival counters, NBUF completion counters
    static constexpr int flags = cnt + (2 * NBUF + NSTAGE) * 4;      // + down: NSTAGE stage-free counters
    static constexpr int total = flags + 16;
};

// ---------------------------------------------------------------------------------------------------------------------
// prepare (the device code is in hmoe_prepare.cuh; the router can run it inside its own launch instead)
__global__ void __launch_bounds__(256) decode_prepare_kernel(const void* __restrict__ x, int x_kind, const int64_t* __restrict__ sel,
    const __half* __restrict__ rw, int R, int H, int topk, int lo, int n_local, int has_shared, int act_quant,
    __half* __restrict__ xf, float* __restrict__ xscale, Route* __restrict__ route, int sh_mod, int sh_rem, unsigned* gen_bump,
    float4* __restrict__ gzero, int gzero_n, int I, int nblocks)
{
    __shared__ RouteSmem S;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");      // the next kernel's blocks may set up while this one runs
    if ((int) blockIdx.x < R) prepare_row(x, x_kind, blockIdx.x, H, act_quant, xf, xscale, gzero, gzero_n, threadIdx.x, blockDim.x);
    else build_route<false>(S, sel, rw, R, H, I, topk, lo, n_local, has_shared, sh_mod, sh_rem, gen_bump, route, nblocks, threadIdx.x);
}

// Set-up step of a short-prefill call: blocks 0 .. R-1 rewrite one row each exactly like the decode set-up; the last block
// builds the tile list from the selections. The picks are counted per expert with shared-memory atomics; one warp turns the
// counts into prefix sums (first tile, first row of the per-pick buffer, cost before the expert's items); every expert's
// thread writes the headers of its tiles; one warp then walks the picks in order, 32 at a time (lanes with the same expert
// find each other with a match, the expert's fill count moves on by the size of the group), and writes every pick into its
// tile column. Tiles therefore come in ascending expert order with their picks in row order, the shared expert last, as in
// a decode call.
constexpr int SHORT_THREADS = 288;          // >= 256 local experts + the shared expert; nine slots per lane in the prefix warp
__global__ void __launch_bounds__(SHORT_THREADS) short_prepare_kernel(const void* __restrict__ x, int x_kind, const int64_t* __restrict__ sel,
    const __half* __restrict__ rw, int R, int H, int topk, int lo, int n_local, int has_shared, int act_quant,
    __half* __restrict__ xf, float* __restrict__ xscale, RouteShort* __restrict__ route, int sh_row0, int sh_rows,
    float4* __restrict__ gzero, int gzero_n, int I, int nblocks)
{
    __shared__ short s_sel[SHORT_MAXR * TOPK_MAX];
    __shared__ int s_n[SHORT_THREADS], s_fill[SHORT_THREADS], s_pre[4][SHORT_THREADS];      // s_pre: tiles, rows, cost in gate_up, cost in down before the slot
    __shared__ int s_cum[2][SHORT_MAXT + 1];
    __shared__ unsigned char s_nn[SHORT_MAXT];
    __shared__ int s_tot[4];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");      // the next kernel's blocks may set up while this one runs
    if ((int) blockIdx.x < R) { prepare_row(x, x_kind, blockIdx.x, H, act_quant, xf, xscale, gzero, gzero_n, threadIdx.x, blockDim.x); return; }
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, P = R * topk, ns = n_local + (has_shared ? 1 : 0);
    const int J0 = 2 * (I / 64), J1 = H / 64;
    // the cost model of the decode set-up: an item of a tile with more real rows issues more reductions
    auto cost0 = [&](int n) { return J0 * ((n >> 3) * 408 + ((n & 7) ? 400 + (n & 7) : 0)); };
    auto cost1 = [&](int n) { return J1 * ((n >> 3) * 124 + ((n & 7) ? 100 + 3 * (n & 7) : 0)); };
    s_n[tid] = 0; s_fill[tid] = 0;
    __syncthreads();
    for (int i = tid; i < P; i += SHORT_THREADS)
    {
        const int64_t e = sel[i] - lo;
        const bool mine = e >= 0 && e < n_local;
        s_sel[i] = mine ? (short) e : (short) -1;
        if (mine) atomicAdd(&s_n[(int) e], 1);
    }
    if (has_shared && tid == 0) s_n[n_local] = sh_rows;                  // the shared expert serves rows [sh_row0, sh_row0 + sh_rows)
    __syncthreads();
    const int n = tid < ns ? s_n[tid] : 0;
    const int m = __syncthreads_count(tid < n_local && n > 0);
    if (warp == 0)
    {
        constexpr int PER = SHORT_THREADS / 32;
        int v[4] = {0, 0, 0, 0};
        #pragma unroll
        for (int k = 0; k < PER; ++k)
        {
            const int e = lane * PER + k, ne = e < ns ? s_n[e] : 0;
            v[0] += (ne + 7) >> 3; v[1] += ne; v[2] += cost0(ne); v[3] += cost1(ne);
        }
        int incl[4] = {v[0], v[1], v[2], v[3]};
        #pragma unroll
        for (int o = 1; o < 32; o <<= 1)
            #pragma unroll
            for (int c = 0; c < 4; ++c) { const int t = __shfl_up_sync(0xffffffffu, incl[c], o); if (lane >= o) incl[c] += t; }
        int run[4] = {incl[0] - v[0], incl[1] - v[1], incl[2] - v[2], incl[3] - v[3]};
        #pragma unroll
        for (int k = 0; k < PER; ++k)
        {
            const int e = lane * PER + k, ne = e < ns ? s_n[e] : 0;
            #pragma unroll
            for (int c = 0; c < 4; ++c) s_pre[c][e] = run[c];
            run[0] += (ne + 7) >> 3; run[1] += ne; run[2] += cost0(ne); run[3] += cost1(ne);
        }
        if (lane == 31)
            #pragma unroll
            for (int c = 0; c < 4; ++c) s_tot[c] = incl[c];
    }
    __syncthreads();
    const int nt = s_tot[0], t0 = s_pre[0][tid];
    if (tid == 0)
    {
        route->m = m; route->ntiles = nt; route->pad[0] = route->pad[1] = 0;
        s_cum[0][nt] = s_tot[2]; s_cum[1][nt] = s_tot[3];
    }
    if (n > 0)
    {
        int c0 = s_pre[2][tid], c1 = s_pre[3][tid];
        const int rb = s_pre[1][tid];
        for (int b8 = 0, t = t0; b8 < n; b8 += 8, ++t)
        {
            const int nn = n - b8 < 8 ? n - b8 : 8;
            route->expert[t] = tid < n_local ? (short) tid : (short) -1; route->nrows[t] = (unsigned char) nn; route->rowbase[t] = (short) (rb + b8);
            s_nn[t] = (unsigned char) nn; s_cum[0][t] = c0; s_cum[1][t] = c1;
            c0 += J0 * (400 + nn); c1 += J1 * (100 + 3 * nn);
        }
    }
    if (warp == 1)
    {
        for (int base = 0; base < P; base += 32)
        {
            const int i = base + lane, e = i < P ? (int) s_sel[i] : -1;
            const unsigned peers = __match_any_sync(0xffffffffu, e), before = peers & ((1u << lane) - 1u);
            if (e >= 0)
            {
                const int pos = s_fill[e] + __popc(before), t = s_pre[0][e] + (pos >> 3), c = pos & 7;
                route->rows[t][c] = (unsigned short) (i / topk); route->w[t][c] = __half2float(rw[i]);
            }
            __syncwarp();
            if (e >= 0 && before == 0) s_fill[e] += __popc(peers);        // the first lane of every group moves the expert's fill count on
            __syncwarp();
        }
    }
    else if (warp == 2 && has_shared)
    {
        for (int pos = lane; pos < sh_rows; pos += 32)
        {
            const int t = s_pre[0][n_local] + (pos >> 3), c = pos & 7;
            route->rows[t][c] = (unsigned short) (sh_row0 + pos); route->w[t][c] = 1.f;
        }
    }
    __syncthreads();
    // columns beyond the picks of an expert's last tile: the tile's first row again, weight 0 (computed, never written out)
    if (n & 7)
    {
        const int t = t0 + (n >> 3);
        const unsigned short first = route->rows[t][0];
        for (int c = n & 7; c < 8; ++c) { route->rows[t][c] = first; route->w[t][c] = 0.f; }
    }
    // the blocks' item ranges, cut at equal cost
    for (int i = tid; i < 2 * (nblocks + 1); i += SHORT_THREADS)
    {
        const int k = i / (nblocks + 1), b = i % (nblocks + 1), J = k ? J1 : J0;
        int p = nt * J;
        if (b < nblocks && nt > 0)
        {
            const int target = (int) ((long long) s_cum[k][nt] * b / nblocks);
            int lo2 = 0, hi = nt - 1;                    // last tile whose start is <= target
            while (lo2 < hi) { const int mid = (lo2 + hi + 1) >> 1; if (s_cum[k][mid] <= target) lo2 = mid; else hi = mid - 1; }
            const int item = k ? 100 + 3 * s_nn[lo2] : 400 + s_nn[lo2];
            const int off = (target - s_cum[k][lo2]) / item;
            p = lo2 * J + (off < J ? off : J);
        }
        route->split[k][b] = p;
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// What a warp needs from global memory for its two 64-column blocks (one 128-column scale group) of a ring stage,
// fetched one stage ahead.
struct Pre
{
    uint32_t bx[2][8];      // activation fragments of this lane's tile row per block: word 2t + h of 16-column step t
    uint4 sc;               // GROUPED: bf16 scales of rows strip*16 + g (low half of word `strip`) and + 8 (high half)
    float4 sx[2];           // Q8: activation scales of the group's four 32-column quarters for tile columns 2q and 2q + 1
};

// The expert-parallel combine, done by the down launch itself when its blocks run out of weights to stream (instead of a kernel
// of its own after it). The block that finishes last raises this rank's generation in every peer's flag array (release, system
// scope); every block then waits, bounded, until all peers have raised theirs here, and sums its slice of the peers' partial slots
// into the layer output in rank order (all rows: identical bits on every rank; or only the rows this rank owns when the tokens
// are data-parallel), and clears its slice of the other slot for the step after next. Blocks that finish early wait on SMs that
// would otherwise idle: the tail costs one flag round trip and one round of peer loads after the slowest rank's last weight.
struct EpTail
{
    int rank, world, own_rows, n;     // n = rows * H
    float* slots[8];                  // slots[p] = rank p's two partial slots as seen from here
    unsigned* flags[8];               // flags[p] = rank p's flag array [world]
    float* f;                         // layer output, added into
    unsigned* done;                   // arrival counter of this launch's blocks (in the workspace, returns to zero)
    unsigned* status;                 // status word for a wait that gives up
};

__device__ __forceinline__ void ep_st_release_sys(unsigned* p, unsigned v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ unsigned ep_ld_acquire_sys(const unsigned* p)
{
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float4 ep_ld_peer(const float4* p)
{
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}

// called by all threads of every block of the down launch, after the block's last reduction has been issued
__device__ __forceinline__ void ep_tail_combine(const EpTail& e, unsigned gen, size_t slot_floats, int H)
{
    __shared__ int ok_sh;
    __syncthreads();
    if (threadIdx.x == 0)
    {
        __threadfence();
        if (atomicAdd(e.done, 1u) == gridDim.x - 1)
        {
            *e.done = 0u;
            __threadfence_system();
            for (int p = 0; p < e.world; ++p) ep_st_release_sys(e.flags[p] + e.rank, gen);
        }
        int ok = 1;
        const unsigned long long t0 = globaltimer_ns();
        for (int p = 0; p < e.world && ok; ++p)
            while ((int) (ep_ld_acquire_sys(e.flags[e.rank] + p) - gen) < 0)
                if (globaltimer_ns() - t0 > 2000000000ull) { ok = 0; atomicOr(e.status, ST_WAIT_TIMEOUT); break; }
        ok_sh = ok;
    }
    __syncthreads();
    if (!ok_sh) return;
    const int parity = gen & 1;
    for (int i = (blockIdx.x * blockDim.x + threadIdx.x) * 4; i < e.n; i += gridDim.x * blockDim.x * 4)
    {
        *(float4*) (e.slots[e.rank] + (size_t) (parity ^ 1) * slot_floats + i) = make_float4(0.f, 0.f, 0.f, 0.f);
        int o = i;
        if (e.own_rows)
        {
            const int r = i / H;
            if (r % e.world != e.rank) continue;
            o = (r / e.world) * H + (i - r * H);
        }
        // all peers' loads are issued before the first sum (a warp issues in order: a sum between two loads would serialise
        // the NVLink round trips); the sums then run in rank order
        float4 v[8];
        #pragma unroll
        for (int p = 0; p < 8; ++p)
            if (p < e.world) v[p] = ep_ld_peer((const float4*) (e.slots[p] + (size_t) parity * slot_floats + i));
        float4 acc = *(float4*) (e.f + o);
        #pragma unroll
        for (int p = 0; p < 8; ++p)
            if (p < e.world) { acc.x += v[p].x; acc.y += v[p].y; acc.z += v[p].z; acc.w += v[p].w; }
        *(float4*) (e.f + o) = acc;
    }
}

struct DecodeArgs
{
    int H, I;
    const int64_t* gate_w; const int64_t* up_w; const int64_t* down_w;
    const int64_t* gate_s; const int64_t* up_s; const int64_t* down_s;
    const void* sh_gw; const void* sh_uw; const void* sh_dw; const void* sh_gs; const void* sh_us; const void* sh_ds;
    const Route* route;
    const __half* xf;      // [R][H] prepared rows
    const float* xscale;   // [R][H/32] (Q8)
    __half* act;           // [tiles][8][I] gate_up output = down input
    float* ascale;         // [tiles][8][I/32] (Q8)
    float* G;              // I <= 2048 path: [pick rows][gate | up][I] fp32 sums (shares memory with act)
    float* y;              // [R][H] (expert-parallel: base of two slots, the step's slot is chosen by *gen_ptr & 1)
    const unsigned* gen_ptr; size_t slot_stride;
    unsigned* status;
    EpTail ep;             // expert parallel: the combine over peer memory as the tail of the down launch (world = 0: none)
};

// Two 64-column blocks (one scale group) of a 64-row group: 4 strips x 8 steps of MMAs on the tile, added into acc with
// the scales applied. wsm = shared address of the first block's 2 KB unit; the second follows it.
template <bool GROUPED, bool Q8>
__device__ __forceinline__ void consume_group(uint32_t wsm, const uint32_t (&bx)[2][8], const uint4 sc, const float4 sx0, const float4 sx1,
                                              float (*acc)[4], int lane)
{
    const uint32_t scw[4] = {sc.x, sc.y, sc.z, sc.w};
    const float sxa[4] = {sx0.x, sx0.y, sx0.z, sx0.w}, sxb[4] = {sx1.x, sx1.y, sx1.z, sx1.w};
    // The four strips' sums are independent MMA chains; the steps are interleaved across strips so that consecutive MMAs
    // never wait on each other.
    float part[4][4];
    #pragma unroll
    for (int s = 0; s < 4; ++s) part[s][0] = part[s][1] = part[s][2] = part[s][3] = 0.f;
    #pragma unroll
    for (int blk = 0; blk < 2; ++blk)
    {
        uint4 w4[4];
        #pragma unroll
        for (int s = 0; s < 4; ++s) w4[s] = lds128(wsm + blk * 2048 + s * 512 + lane * 16);
        #pragma unroll
        for (int t = 0; t < 4; ++t)
        {
            #pragma unroll
            for (int s = 0; s < 4; ++s)
            {
                const uint32_t w = t == 0 ? w4[s].x : t == 1 ? w4[s].y : t == 2 ? w4[s].z : w4[s].w;
                uint32_t a[4];
                frag_from_codes(w, a);
                mma_f16((GROUPED || Q8) ? part[s] : acc[s], a, bx[blk][2 * t], bx[blk][2 * t + 1]);
            }
            if (Q8 && (t & 1))
            {
                // int8 activations: the sums of 32 columns are exact integers; one multiply by (activation scale x weight scale)
                const int qt = blk * 2 + (t >> 1);
                #pragma unroll
                for (int s = 0; s < 4; ++s)
                {
                    float s0 = 1.f, s1 = 1.f;
                    if (GROUPED) { s0 = __uint_as_float(scw[s] << 16); s1 = __uint_as_float(scw[s] & 0xffff0000u); }
                    acc[s][0] = fmaf(part[s][0], sxa[qt] * s0, acc[s][0]); acc[s][1] = fmaf(part[s][1], sxb[qt] * s0, acc[s][1]);
                    acc[s][2] = fmaf(part[s][2], sxa[qt] * s1, acc[s][2]); acc[s][3] = fmaf(part[s][3], sxb[qt] * s1, acc[s][3]);
                    part[s][0] = part[s][1] = part[s][2] = part[s][3] = 0.f;
                }
            }
        }
    }
    if (GROUPED && !Q8)
    {
        #pragma unroll
        for (int s = 0; s < 4; ++s)
        {
            const float s0 = __uint_as_float(scw[s] << 16), s1 = __uint_as_float(scw[s] & 0xffff0000u);
            acc[s][0] = fmaf(s0, part[s][0], acc[s][0]); acc[s][1] = fmaf(s0, part[s][1], acc[s][1]);
            acc[s][2] = fmaf(s1, part[s][2], acc[s][2]); acc[s][3] = fmaf(s1, part[s][3], acc[s][3]);
        }
    }
}

// what a lane keeps about the item it is working on
struct Item
{
    int tile, gr, e, nrows;
    const char* xb;         // this lane's activation row, offset to its 32-byte chunk of block 0
    const float* xs[2];     // Q8: activation scale rows of tile columns 2q, 2q + 1
    const char* sc;         // GROUPED: scale words of this lane's rows for the item's 64-row group (column group 0)
};

// kb = first of the warp's two blocks (even)
template <bool GROUPED, bool Q8>
__device__ __forceinline__ void prefetch(const Item& it, int kb, int KB, Pre& pr)
{
    if (kb >= KB) return;
    const uint4 b0 = ldg128(it.xb + kb * 128), b1 = ldg128(it.xb + kb * 128 + 16);
    const uint4 b2 = ldg128(it.xb + kb * 128 + 128), b3 = ldg128(it.xb + kb * 128 + 144);
    pr.bx[0][0] = b0.x; pr.bx[0][1] = b0.y; pr.bx[0][2] = b0.z; pr.bx[0][3] = b0.w;
    pr.bx[0][4] = b1.x; pr.bx[0][5] = b1.y; pr.bx[0][6] = b1.z; pr.bx[0][7] = b1.w;
    pr.bx[1][0] = b2.x; pr.bx[1][1] = b2.y; pr.bx[1][2] = b2.z; pr.bx[1][3] = b2.w;
    pr.bx[1][4] = b3.x; pr.bx[1][5] = b3.y; pr.bx[1][6] = b3.z; pr.bx[1][7] = b3.w;
    if (Q8) { pr.sx[0] = *(const float4*) (it.xs[0] + 2 * kb); pr.sx[1] = *(const float4*) (it.xs[1] + 2 * kb); }
    if (GROUPED) pr.sc = ldg128_nc(it.sc + (size_t) (kb >> 1) * 128);
}

// Each warp owns a private three-slot ring of 4 KB (its two 64-column blocks of a stage) with one mbarrier per slot. When it
// has read a slot, its lane 0 at once issues the 1-D bulk copy of the data it will need three stages later into that slot,
// so the warps stream independently: nobody waits for the slowest warp of a stage and no slot ever waits to be freed.
// ---------------------------------------------------------------------------------------------------------------------
// gate_up
template <bool GROUPED, bool Q8>
__global__ void __launch_bounds__(NTHREADS, 1) decode_gate_up_kernel(const DecodeArgs a)
{
    extern __shared__ __align__(1024) unsigned char smem[];
    const uint32_t sbase = smem_u32(smem);
    const uint32_t ring = sbase + SmemLayout::ring, full0 = sbase + SmemLayout::bars;
    float* gu = (float*) (smem + SmemLayout::gu);
    int* cnt = (int*) (smem + SmemLayout::cnt);
    volatile int* abort_flag = (volatile int*) (smem + SmemLayout::flags);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0)
    {
        for (int i = 0; i < NSTAGE * CW; ++i) mbar_init(full0 + i * 8, 1);
        for (int i = 0; i < 2 * NBUF; ++i) cnt[i] = 0;
        *abort_flag = 0;
        fence_barrier_init();
    }
    for (int i = threadIdx.x; i < NBUF * GU_FLOATS; i += NTHREADS) gu[i] = 0.f;
    __syncthreads();
    const Route* rt = a.route;
    const int NG = a.I / 64, KB = a.H / 64, S = (KB + 15) / 16;
    const int P = rt->ntiles * NG;
    const int p0 = (int) ((long long) P * blockIdx.x / gridDim.x), p1 = (int) ((long long) P * (blockIdx.x + 1) / gridDim.x);
    const int mat = warp >> 3, kw = warp & 7, g = lane >> 2, q = lane & 3;
    // fill cursor of this warp: the next stage to request is stage f_s of item (f_tile, f_gr); f_src = its matrix's packed codes
    int f_tile = p0 / NG, f_gr = p0 % NG, f_s = 0, f_left = p1 - p0;
    auto item_src = [&](int tile, int gr) {
        const int e = rt->expert[tile];
        return (const char*) (e >= 0 ? (const void*) (mat ? a.up_w[e] : a.gate_w[e]) : (mat ? a.sh_uw : a.sh_gw)) + (size_t) gr * KB * 2048;
    };
    const char* f_src = p0 < p1 ? item_src(f_tile, f_gr) : nullptr;      // looked up when the cursor enters an item, used a stage later
    auto fill_next = [&](uint32_t slot) {
        if (f_left <= 0) return;
        const int kb = 16 * f_s + 2 * kw;
        if (kb < KB)
        {
            const uint32_t bar = full0 + (slot * CW + warp) * 8;
            mbar_expect_tx(bar, 4096);
            bulk_g2s(ring + slot * STAGE_BYTES + warp * 4096, f_src + (size_t) kb * 2048, 4096, bar);
        }
        if (++f_s == S)
        {
            f_s = 0; --f_left;
            if (++f_gr == NG) { f_gr = 0; ++f_tile; }
            if (f_left > 0) f_src = item_src(f_tile, f_gr);
        }
    };
    auto load_item = [&](int tile, int gr) {
        Item it;
        it.tile = tile; it.gr = gr; it.e = rt->expert[it.tile]; it.nrows = rt->nrows[it.tile];
        it.xb = (const char*) (a.xf + (size_t) rt->rows[it.tile][g] * a.H) + q * 32;
        if (Q8)
        {
            it.xs[0] = a.xscale + (size_t) rt->rows[it.tile][2 * q] * (a.H / 32);
            it.xs[1] = a.xscale + (size_t) rt->rows[it.tile][2 * q + 1] * (a.H / 32);
        }
        if (GROUPED)
        {
            const void* sp = it.e >= 0 ? (const void*) (mat ? a.up_s[it.e] : a.gate_s[it.e]) : (mat ? a.sh_us : a.sh_gs);
            it.sc = (const char*) sp + ((size_t) it.gr * (a.H / 128) * 64 + g * 8) * 2;
        }
        return it;
    };
    if (p0 < p1)
    {
        if (lane == 0)
            for (uint32_t i = 0; i < NSTAGE; ++i) fill_next(i);
        float acc[4][4];
        #pragma unroll
        for (int i = 0; i < 4; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
        Item cur = load_item(p0 / NG, p0 % NG);
        Pre pc;
        prefetch<GROUPED, Q8>(cur, 2 * kw, KB, pc);
        uint32_t it = 0, st = 0, par = 0;
        bool alive = true;
        // Finishing an item: warp w owns tile column w / 2 and rows 32 (w % 2) + lane of the 64-row group. It waits (bounded)
        // until all CW partial tiles of the item are in, reads its gate / up sums, clears them for the buffer's next use and
        // writes act = silu(gate) * up * routing weight as the down kernel's MMA operand. A warp does this one ring stage
        // after it delivered its own partial; it
        // counts itself done afterwards, and no warp adds a later item's partial into the buffer before all sixteen are done
        // with the buffer's previous item (the warps stream independently and may drift apart).
        Item prev = cur; bool have_prev = false; int prev_idx = 0;
        auto finish_item = [&](const Item& pi, int idx) {
            const int b = idx % NBUF, target = CW * (idx / NBUF + 1);
            volatile int* c = cnt + b;
            if (*c < target)
            {
                const unsigned long long t0 = globaltimer_ns();
                while (*c < target)
                    if (globaltimer_ns() - t0 > 1000000000ull) { *abort_flag = 1; atomicOr(a.status, ST_WAIT_TIMEOUT); break; }
            }
            __threadfence_block();
            const int col = warp >> 1, n = (warp & 1) * 32 + lane;
            float* g0 = gu + b * GU_FLOATS;
            float gg = g0[n * 8 + col], uu = g0[512 + n * 8 + col];
            g0[n * 8 + col] = 0.f; g0[512 + n * 8 + col] = 0.f;
            float v = 0.f;
            if (col < pi.nrows)
            {
                if (!GROUPED)
                {
                    const float* gsp = pi.e >= 0 ? (const float*) a.gate_s[pi.e] : (const float*) a.sh_gs;
                    const float* usp = pi.e >= 0 ? (const float*) a.up_s[pi.e] : (const float*) a.sh_us;
                    gg *= __ldg(gsp + pi.gr * 64 + n); uu *= __ldg(usp + pi.gr * 64 + n);
                }
                v = gg / (1.f + expf(-gg)) * uu * rt->w[pi.tile][col];
            }
            const size_t row = (size_t) pi.tile * 8 + col;
            if (Q8)
            {
                // second int8 round trip of the CPU engine (cpuband.cpp:200-207): 32 consecutive outputs = this warp
                float m = fabsf(v);
                #pragma unroll
                for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
                const float sc = m > 0.f ? __fdiv_rn(m, 127.f) : 1.f;
                v = (float) __float2int_rn(__fmul_rn(v, __fdiv_rn(1.f, sc)));
                if (lane == 0) a.ascale[row * (a.I / 32) + pi.gr * 2 + (warp & 1)] = sc;
            }
            a.act[row * a.I + pi.gr * 64 + frag_pos(n >> 1) * 2 + (n & 1)] = __float2half_rn(v);
            __syncwarp();
            if (lane == 0) { __threadfence_block(); atomicAdd(cnt + NBUF + b, 1); }
        };
        for (int p = p0; p < p1 && alive; ++p)
        {
            Item nxt = cur;
            for (int s = 0; s < S; ++s, ++it)
            {
                Pre pn = pc;
                if (s + 1 < S) prefetch<GROUPED, Q8>(cur, 16 * (s + 1) + 2 * kw, KB, pn);
                else if (p + 1 < p1)
                {
                    const bool wrap = cur.gr + 1 == NG;
                    nxt = load_item(wrap ? cur.tile + 1 : cur.tile, wrap ? 0 : cur.gr + 1);
                    prefetch<GROUPED, Q8>(nxt, 2 * kw, KB, pn);
                }
                if (16 * s + 2 * kw < KB)
                {
                    if (!mbar_wait(full0 + (st * CW + warp) * 8, par, abort_flag, a.status)) { alive = false; break; }
                    consume_group<GROUPED, Q8>(ring + st * STAGE_BYTES + warp * 4096, pc.bx, pc.sc, pc.sx[0], pc.sx[1], acc, lane);
                }
                __syncwarp();
                if (lane == 0) fill_next(st);
                if (s == 0 && have_prev) { finish_item(prev, prev_idx); have_prev = false; }
                if (++st == NSTAGE) { st = 0; par ^= 1; }
                pc = pn;
            }
            if (!alive) break;
            // This warp's partial tile joins the item's sums in shared memory (buffer b, counted arrivals). Every warp later
            // finishes its own 32 outputs of the item (see finish_item) once all sixteen partials are in.
            const int b = (p - p0) % NBUF;
            {
                volatile int* dc = cnt + NBUF + b;
                const int need = CW * ((p - p0) / NBUF);                  // completions of the buffer's earlier items
                if (*dc < need)
                {
                    const unsigned long long t0 = globaltimer_ns();
                    while (*dc < need)
                        if (globaltimer_ns() - t0 > 1000000000ull) { *abort_flag = 1; atomicOr(a.status, ST_WAIT_TIMEOUT); break; }
                }
                __threadfence_block();
            }
            float* gb = gu + b * GU_FLOATS + mat * 512;
            #pragma unroll
            for (int ss = 0; ss < 4; ++ss)
            {
                atomicAdd(gb + (ss * 16 + g) * 8 + 2 * q, acc[ss][0]); atomicAdd(gb + (ss * 16 + g) * 8 + 2 * q + 1, acc[ss][1]);
                atomicAdd(gb + (ss * 16 + g + 8) * 8 + 2 * q, acc[ss][2]); atomicAdd(gb + (ss * 16 + g + 8) * 8 + 2 * q + 1, acc[ss][3]);
                acc[ss][0] = acc[ss][1] = acc[ss][2] = acc[ss][3] = 0.f;
            }
            __syncwarp();
            if (lane == 0) { __threadfence_block(); atomicAdd(cnt + b, 1); }
            prev = cur; have_prev = true; prev_idx = p - p0;
            cur = nxt;
        }
        if (alive && have_prev) finish_item(prev, prev_idx);
    }
    __syncthreads();
}

// down's ring is shared by the block and refilled by whichever warp frees a stage last: after its last read of stage number `it` a warp bumps the
// stage's counter, and the warp that brings it to CW issues the copies of stage number it + NSTAGE into the same slot.
// No thread ever waits for a free slot.
template <typename Fill>
__device__ __forceinline__ void release_stage(int* free_cnt, uint32_t st, uint32_t it, uint32_t total, int lane, Fill fill)
{
    __syncwarp();
    if (lane == 0)
    {
        __threadfence_block();
        if (atomicAdd(free_cnt + st, 1) == CW - 1)
        {
            free_cnt[st] = 0;
            __threadfence_block();
            if (it + NSTAGE < total) fill(it + NSTAGE);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// down
template <bool GROUPED, bool Q8>
__global__ void __launch_bounds__(NTHREADS, 1) decode_down_kernel(const DecodeArgs a, int R)
{
    extern __shared__ __align__(1024) unsigned char smem[];
    const uint32_t sbase = smem_u32(smem);
    const uint32_t ring = sbase + SmemLayout::ring, full0 = sbase + SmemLayout::bars;
    float* yacc = (float*) (smem + SmemLayout::gu);
    float* const yout = a.y + (a.gen_ptr ? (size_t) (*a.gen_ptr & 1u) * a.slot_stride : 0);
    int* free_cnt = (int*) (smem + SmemLayout::cnt) + 2 * NBUF;
    volatile int* abort_flag = (volatile int*) (smem + SmemLayout::flags);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0)
    {
        for (int i = 0; i < NSTAGE; ++i) mbar_init(full0 + i * 8, 1);
        for (int i = 0; i < NSTAGE; ++i) free_cnt[i] = 0;
        *abort_flag = 0;
        fence_barrier_init();
    }
    for (int i = threadIdx.x; i < 4 * YACC_FLOATS; i += blockDim.x) yacc[i] = 0.f;   // four copies (less contention)
    __syncthreads();
    const Route* rt = a.route;
    const int NG = a.H / 64, KB = a.I / 64, S = (KB + 31) / 32;
    const int nt = rt->ntiles;
    const int P = nt * NG;
    const int p0 = (int) ((long long) P * blockIdx.x / gridDim.x), p1 = (int) ((long long) P * (blockIdx.x + 1) / gridDim.x);
    const int g = lane >> 2, q = lane & 3;
    const uint32_t total = (uint32_t) (p1 - p0) * S;
    auto fill = [&](uint32_t i) {
        const int p = p0 + (int) (i / S), s = (int) (i % S);
        const int gr = p / nt, tile = p % nt, e = rt->expert[tile];
        const char* dw = (const char*) (e >= 0 ? (const void*) a.down_w[e] : a.sh_dw) + ((size_t) gr * KB + 32 * s) * 2048;
        const uint32_t st = i % NSTAGE, bytes = (KB - 32 * s < 32 ? KB - 32 * s : 32) * 2048;
        mbar_expect_tx(full0 + st * 8, bytes);
        bulk_g2s(ring + st * STAGE_BYTES, dw, bytes, full0 + st * 8);
    };
    auto load_item = [&](int gr, int tile) {
        Item it;
        it.gr = gr; it.tile = tile; it.e = rt->expert[it.tile]; it.nrows = rt->nrows[it.tile];
        const size_t trow = (size_t) it.tile * 8;
        it.xb = (const char*) (a.act + (trow + g) * a.I) + q * 32;
        if (Q8) { it.xs[0] = a.ascale + (trow + 2 * q) * (a.I / 32); it.xs[1] = a.ascale + (trow + 2 * q + 1) * (a.I / 32); }
        if (GROUPED)
        {
            const void* sp = it.e >= 0 ? (const void*) a.down_s[it.e] : a.sh_ds;
            it.sc = (const char*) sp + ((size_t) it.gr * (a.I / 128) * 64 + g * 8) * 2;
        }
        return it;
    };
    if (p0 < p1)
    {
        if (threadIdx.x == 0)
            for (uint32_t i = 0; i < NSTAGE && i < total; ++i) fill(i);
        float acc[4][4];
        #pragma unroll
        for (int i = 0; i < 4; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
        Item cur = load_item(p0 / nt, p0 % nt);
        Pre pc;
        prefetch<GROUPED, Q8>(cur, 2 * warp, KB, pc);
        uint32_t it = 0, st = 0, par = 0;
        bool alive = true;
        for (int p = p0; p < p1 && alive; ++p)
        {
            Item nxt = cur;
            for (int s = 0; s < S; ++s, ++it)
            {
                Pre pn = pc;
                if (s + 1 < S) prefetch<GROUPED, Q8>(cur, 32 * (s + 1) + 2 * warp, KB, pn);
                else if (p + 1 < p1)
                {
                    const bool wrap = cur.tile + 1 == nt;
                    nxt = load_item(wrap ? cur.gr + 1 : cur.gr, wrap ? 0 : cur.tile + 1);
                    prefetch<GROUPED, Q8>(nxt, 2 * warp, KB, pn);
                }
                if (!mbar_wait(full0 + st * 8, par, abort_flag, a.status)) { alive = false; break; }
                if (32 * s + 2 * warp < KB) consume_group<GROUPED, Q8>(ring + st * STAGE_BYTES + warp * 4096, pc.bx, pc.sc, pc.sx[0], pc.sx[1], acc, lane);
                release_stage(free_cnt, st, it, total, lane, fill);
                if (++st == NSTAGE) { st = 0; par ^= 1; }
                pc = pn;
            }
            if (!alive) break;
            float sd[8];
            #pragma unroll
            for (int i = 0; i < 8; ++i) sd[i] = 1.f;
            if (!GROUPED)
            {
                const float* dsp = cur.e >= 0 ? (const float*) a.down_s[cur.e] : (const float*) a.sh_ds;
                #pragma unroll
                for (int ss = 0; ss < 4; ++ss) { sd[2 * ss] = __ldg(dsp + cur.gr * 64 + ss * 16 + g); sd[2 * ss + 1] = __ldg(dsp + cur.gr * 64 + ss * 16 + g + 8); }
            }
            // add this warp's share of the tile's contribution into the block's slice of y, real row by real row
            #pragma unroll
            for (int c = 0; c < 2; ++c)
            {
                const int col = 2 * q + c;
                if (col < cur.nrows)
                {
                    float* yr = yacc + (warp >> 2) * YACC_FLOATS + (int) rt->rows[cur.tile][col] * 64;
                    #pragma unroll
                    for (int ss = 0; ss < 4; ++ss)
                    {
                        atomicAdd(yr + ss * 16 + g, acc[ss][c] * sd[2 * ss]);
                        atomicAdd(yr + ss * 16 + g + 8, acc[ss][2 + c] * sd[2 * ss + 1]);
                    }
                }
            }
            #pragma unroll
            for (int ss = 0; ss < 4; ++ss) acc[ss][0] = acc[ss][1] = acc[ss][2] = acc[ss][3] = 0.f;
            if (p + 1 >= p1 || cur.tile + 1 == nt)
            {
                // the slice of y this block has been adding into is complete: one fp32 reduction per element to global
                __syncthreads();
                for (int i = threadIdx.x; i < R * 64; i += NTHREADS)
                {
                    const float v = (yacc[i] + yacc[YACC_FLOATS + i]) + (yacc[2 * YACC_FLOATS + i] + yacc[3 * YACC_FLOATS + i]);
                    if (v != 0.f) atomicAdd(yout + (size_t) (i >> 6) * a.H + cur.gr * 64 + (i & 63), v);
                    yacc[i] = yacc[YACC_FLOATS + i] = yacc[2 * YACC_FLOATS + i] = yacc[3 * YACC_FLOATS + i] = 0.f;
                }
                __syncthreads();
            }
            cur = nxt;
        }
    }
    __syncthreads();
}

// ---------------------------------------------------------------------------------------------------------------------
// The streaming kernel of the H <= 6144, I <= 2048 path, used twice per call: gate_up (DOWN = false) and down (DOWN = true).
//
// An item is (tile, matrix, 64-row group of the output): 64 rows x all K input columns of codes (gate_up: 192 KB for
// K = 6144, down: 64 KB). Items are dealt out to the blocks as contiguous ranges with the row group fastest, then the
// matrix (gate, up), then the tile, so a block walks the matrices in address order and stays with one tile - one set of
// activations - for a long time. The K columns are cut into KC chunks of 2048; warp w owns the 128 columns
// [2048 kc + 128 w, + 128) of every chunk: one scale group, 4 KB of codes, contiguous in memory. Its activation fragments
// for those columns (16 registers per chunk) stay in registers for the whole tile, so the inner loop reads nothing but
// shared memory. Every warp has a private ring of NSTAGE slots (4 KB of codes + the 128 bytes of bf16 scales of the same
// 64 rows x 128 columns), each with its own mbarrier; when the warp has read a slot its lane 0 at once issues the copies
// for the slot's next use, so the warps stream independently and no warp ever waits for another.
// A warp ends an item with a 64 x 8 partial tile over its KC x 128 columns; the real tile columns are added to the result
// with fp32 reductions in global memory (sixteen per output element, one per warp):
//   gate_up -> G[pick row][gate | up][I]  (zeroed by the prepare kernel; pick row = Route::rowbase[tile] + tile column)
//   down    -> y[row][H]
// Between the two launches nothing else runs: the down kernel turns G into its own MMA operand when it enters a tile
// (SiLU(gate) * up * routing weight, in the int8 mode followed by the CPU engine's second int8 round trip).
// Programmatic dependent launch: a kernel lets the next one in the stream start as its own blocks retire (the next kernel's
// blocks set up their barriers and request their first weights meanwhile), and the next kernel waits here for the full
// completion of its predecessor, memory included, before it reads anything the predecessor wrote. Both are no-ops for a
// kernel launched without the attribute.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ void red_add(float* p, float v)
{
    asm volatile("red.global.add.f32 [%0], %1;" ::"l"(__cvta_generic_to_global(p)), "f"(v) : "memory");
}

struct StreamSmem
{
    static constexpr int SLOT = 4096 + 128;
    static constexpr int bars = NSTAGE * CW * SLOT;
    static constexpr int flags = bars + NSTAGE * CW * 8;
    static constexpr int total = flags + 16;
};

template <bool GROUPED, bool Q8, bool DOWN, int KC, typename RT = Route>
__global__ void __launch_bounds__(NTHREADS, 1) decode_stream_kernel(const DecodeArgs a)
{
    extern __shared__ __align__(1024) unsigned char smem[];
    constexpr int SLOT = StreamSmem::SLOT;
    const uint32_t sbase = smem_u32(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
    const uint32_t ring = sbase + warp * SLOT, full0 = sbase + StreamSmem::bars + warp * 8;      // slot st: + st * CW * SLOT / + st * CW * 8
    volatile int* abort_flag = (volatile int*) (smem + StreamSmem::flags);
    if (threadIdx.x == 0)
    {
        for (int i = 0; i < NSTAGE * CW; ++i) mbar_init(sbase + StreamSmem::bars + i * 8, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();
    // gate_up follows the prepare kernel, which wrote the route; down follows gate_up, but the route and the weights it
    // needs to fill its rings are older than that: it waits only before it reads the gate / up sums.
    // Ordering rule of the chain: a kernel lets its dependents start only after its own wait has returned, i.e. after the
    // kernel before it has completed with its memory visible. So whatever a dependent reads before ITS wait (down: the route,
    // the step counter) was written at least two kernels back and is complete, whatever the occupancy. Blocks without work
    // wait too, so that a grid with nothing to do cannot release its dependents early.
    TL_MIN(DOWN ? 8 : 0);
    if (!DOWN) { pdl_wait(); pdl_launch_dependents(); TL_MIN(2); }
    const RT* rt = reinterpret_cast<const RT*>(a.route);          // RT = RouteShort: the same fields with room for more tiles
    const int K = DOWN ? a.I : a.H, N = DOWN ? a.H : a.I;          // input columns and output rows of one matrix
    const int KB = K / 64, NG = N / 64, J = DOWN ? NG : 2 * NG;
    const int p0 = rt->split[DOWN][blockIdx.x], p1 = rt->split[DOWN][blockIdx.x + 1];      // cut at equal cost by the prepare kernel
    float* const out0 = DOWN ? a.y + (a.gen_ptr ? (size_t) (*a.gen_ptr & 1u) * a.slot_stride : 0) : a.G;
    if (p0 < p1 && 2 * warp < KB)
    {
        // ---- fill cursor (lane 0): the next slot to request is chunk f_kc of item (f_tile, f_j)
        int f_p = p0, f_tile = p0 / J, f_j = p0 % J, f_kc = 0;
        const char* f_w = nullptr; const char* f_s = nullptr;
        auto fill_next = [&](uint32_t slot) {
            if (f_p >= p1) return;
            const int mat = (!DOWN && f_j >= NG) ? 1 : 0, gr = f_j - mat * NG;
            if (f_w == nullptr || (gr == 0 && f_kc == 0))
            {
                const int e = rt->expert[f_tile];
                const void* w = DOWN ? (e >= 0 ? (const void*) a.down_w[e] : a.sh_dw)
                                     : (mat ? (e >= 0 ? (const void*) a.up_w[e] : a.sh_uw) : (e >= 0 ? (const void*) a.gate_w[e] : a.sh_gw));
                f_w = (const char*) w + (size_t) warp * 4096;
                if (GROUPED)
                {
                    const void* sc = DOWN ? (e >= 0 ? (const void*) a.down_s[e] : a.sh_ds)
                                          : (mat ? (e >= 0 ? (const void*) a.up_s[e] : a.sh_us) : (e >= 0 ? (const void*) a.gate_s[e] : a.sh_gs));
                    f_s = (const char*) sc + (size_t) warp * 128;
                }
            }
            const uint32_t bar = full0 + slot * CW * 8, dst = ring + slot * CW * SLOT;
            mbar_expect_tx(bar, GROUPED ? SLOT : 4096);
            bulk_g2s(dst, f_w + ((size_t) gr * KB + f_kc * 32) * 2048, 4096, bar);
            if (GROUPED) bulk_g2s(dst + 4096, f_s + ((size_t) gr * (K / 128) + f_kc * 16) * 128, 128, bar);
            if (++f_kc == KC || f_kc * 32 + 2 * warp >= KB)
            {
                f_kc = 0; ++f_p;
                if (++f_j == J) { f_j = 0; ++f_tile; f_w = nullptr; }
            }
        };
        if (lane == 0)
            for (uint32_t i = 0; i < NSTAGE; ++i) fill_next(i);

        // ---- consume (all lanes)
        uint32_t bx[KC][2][8];                  // the tile's activation fragments of this warp's columns
        float4 sx[KC][2];                       // Q8: their scales per 32 columns for tile columns 2q and 2q + 1
        #pragma unroll
        for (int kc = 0; kc < KC; ++kc) sx[kc][0] = sx[kc][1] = make_float4(1.f, 1.f, 1.f, 1.f);
        int nrows = 0;
        float* outA = nullptr; float* outB = nullptr;         // result rows of tile columns 2q and 2q + 1, at this lane's row g
        const float* sdp[2] = {nullptr, nullptr};             // !GROUPED: per-row scales, at this lane's row g
        auto enter_tile = [&](int tile) {
            const int e = rt->expert[tile];
            nrows = rt->nrows[tile];
            if (!DOWN)
            {
                const char* xb = (const char*) (a.xf + (size_t) rt->rows[tile][g] * a.H) + (size_t) warp * 256 + q * 32;
                #pragma unroll
                for (int kc = 0; kc < KC; ++kc)
                {
                    uint4 b0 = make_uint4(0, 0, 0, 0), b1 = b0, b2 = b0, b3 = b0;
                    if (kc * 32 + 2 * warp < KB)
                    {
                        const char* xk = xb + kc * 4096;
                        b0 = ldg128(xk); b1 = ldg128(xk + 16); b2 = ldg128(xk + 128); b3 = ldg128(xk + 144);
                        if (Q8)
                        {
                            sx[kc][0] = *(const float4*) (a.xscale + (size_t) rt->rows[tile][2 * q] * (a.H / 32) + 64 * kc + 4 * warp);
                            sx[kc][1] = *(const float4*) (a.xscale + (size_t) rt->rows[tile][2 * q + 1] * (a.H / 32) + 64 * kc + 4 * warp);
                        }
                    }
                    bx[kc][0][0] = b0.x; bx[kc][0][1] = b0.y; bx[kc][0][2] = b0.z; bx[kc][0][3] = b0.w;
                    bx[kc][0][4] = b1.x; bx[kc][0][5] = b1.y; bx[kc][0][6] = b1.z; bx[kc][0][7] = b1.w;
                    bx[kc][1][0] = b2.x; bx[kc][1][1] = b2.y; bx[kc][1][2] = b2.z; bx[kc][1][3] = b2.w;
                    bx[kc][1][4] = b3.x; bx[kc][1][5] = b3.y; bx[kc][1][6] = b3.z; bx[kc][1][7] = b3.w;
                }
                const size_t rb = (size_t) rt->rowbase[tile] + 2 * q;
                outA = a.G + rb * 2 * a.I + g; outB = outA + 2 * a.I;
                if (!GROUPED)
                {
                    sdp[0] = (const float*) (e >= 0 ? (const void*) a.gate_s[e] : a.sh_gs) + g;
                    sdp[1] = (const float*) (e >= 0 ? (const void*) a.up_s[e] : a.sh_us) + g;
                }
            }
            else
            {
                // The operand of tile column t is computed by the whole warp, lane L taking columns 2L, 2L + 1 of each of the
                // warp's two blocks (= word L of the block), and handed to the lanes g == t in the order the MMAs read:
                // word [blk][2t' + h] of lane (g, q) is word 8t' + 4h + q of the block.
                #pragma unroll
                for (int blk = 0; blk < 2; ++blk)
                    #pragma unroll
                    for (int wd = 0; wd < 8; ++wd) bx[0][blk][wd] = 0u;
                float sa[4] = {1.f, 1.f, 1.f, 1.f}, sb[4] = {1.f, 1.f, 1.f, 1.f};
                const float* gp = a.G + (size_t) rt->rowbase[tile] * 2 * a.I + (size_t) warp * 128 + 2 * lane;
                for (int t = 0; t < nrows; ++t, gp += 2 * a.I)
                {
                    const float2 g0 = __ldcg((const float2*) gp), g1 = __ldcg((const float2*) (gp + 64));
                    const float2 u0 = __ldcg((const float2*) (gp + a.I)), u1 = __ldcg((const float2*) (gp + a.I + 64));
                    const float wt = rt->w[tile][t];
                    // fp16 operands: the fast exponential is far inside their rounding; the int8 mode follows the CPU engine
                    float v[2][2];
                    v[0][0] = g0.x / (1.f + (Q8 ? expf(-g0.x) : __expf(-g0.x))) * u0.x * wt;
                    v[0][1] = g0.y / (1.f + (Q8 ? expf(-g0.y) : __expf(-g0.y))) * u0.y * wt;
                    v[1][0] = g1.x / (1.f + (Q8 ? expf(-g1.x) : __expf(-g1.x))) * u1.x * wt;
                    v[1][1] = g1.y / (1.f + (Q8 ? expf(-g1.y) : __expf(-g1.y))) * u1.y * wt;
                    #pragma unroll
                    for (int blk = 0; blk < 2; ++blk)
                    {
                        if (Q8)
                        {
                            // second int8 round trip of the CPU engine (cpuband.cpp:200-207): 32 consecutive values = 16 lanes
                            float m = fmaxf(fabsf(v[blk][0]), fabsf(v[blk][1]));
                            #pragma unroll
                            for (int o = 8; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
                            const float sc = m > 0.f ? __fdiv_rn(m, 127.f) : 1.f, inv = __fdiv_rn(1.f, sc);
                            v[blk][0] = (float) __float2int_rn(__fmul_rn(v[blk][0], inv));
                            v[blk][1] = (float) __float2int_rn(__fmul_rn(v[blk][1], inv));
                            // the MMA results of a lane are tile columns 2q and 2q + 1: those lanes keep this column's scales
                            const float s_lo = __shfl_sync(0xffffffffu, sc, 0), s_hi = __shfl_sync(0xffffffffu, sc, 16);
                            if (2 * q == t) { sa[2 * blk] = s_lo; sa[2 * blk + 1] = s_hi; }
                            if (2 * q + 1 == t) { sb[2 * blk] = s_lo; sb[2 * blk + 1] = s_hi; }
                        }
                        const __half2 h = __floats2half2_rn(v[blk][0], v[blk][1]);
                        const uint32_t word = *(const uint32_t*) &h;
                        #pragma unroll
                        for (int wd = 0; wd < 8; ++wd)
                        {
                            const uint32_t got = __shfl_sync(0xffffffffu, word, (wd >> 1) * 8 + (wd & 1) * 4 + q);
                            if (g == t) bx[0][blk][wd] = got;
                        }
                    }
                }
                if (Q8) { sx[0][0] = make_float4(sa[0], sa[1], sa[2], sa[3]); sx[0][1] = make_float4(sb[0], sb[1], sb[2], sb[3]); }
                outA = out0 + (size_t) rt->rows[tile][2 * q] * a.H + g; outB = out0 + (size_t) rt->rows[tile][2 * q + 1] * a.H + g;
                if (!GROUPED) sdp[0] = (const float*) (e >= 0 ? (const void*) a.down_s[e] : a.sh_ds) + g;
            }
        };
        // !GROUPED: the eight per-row scales of this lane's rows for item jj, applied to the finished sums
        auto load_row_scales = [&](int jj, float* sd) {
            const int mat = (!DOWN && jj >= NG) ? 1 : 0, gr = jj - mat * NG;
            #pragma unroll
            for (int i = 0; i < 8; ++i) sd[i] = __ldg(sdp[mat] + gr * 64 + i * 8);
        };
        float sd[8];
        #pragma unroll
        for (int i = 0; i < 8; ++i) sd[i] = 1.f;
        float acc[4][4];
        #pragma unroll
        for (int i = 0; i < 4; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
        uint32_t st = 0, par = 0;
        int tile = p0 / J, j = p0 % J;
        if (DOWN) { pdl_wait(); pdl_launch_dependents(); TL_MIN(10); }
        enter_tile(tile);
        if (!GROUPED) load_row_scales(j, sd);
        bool alive = true;
        for (int p = p0; p < p1 && alive; ++p)
        {
            float sdn[8];
            #pragma unroll
            for (int k = 0; k < 8; ++k) sdn[k] = 1.f;
            const bool same_tile = j + 1 < J;
            if (!GROUPED && same_tile && p + 1 < p1) load_row_scales(j + 1, sdn);          // one item ahead
            #pragma unroll
            for (int kc = 0; kc < KC; ++kc)
            {
                if (kc * 32 + 2 * warp < KB)
                {
                    if (!mbar_wait(full0 + st * CW * 8, par, abort_flag, a.status)) { alive = false; break; }
                    TL_MIN(DOWN ? 12 : 4);
                    const uint32_t slot = ring + st * CW * SLOT;
                    uint4 sc = make_uint4(0, 0, 0, 0);
                    if (GROUPED) sc = lds128(slot + 4096 + g * 16);
                    consume_group<GROUPED, Q8>(slot, bx[kc], sc, sx[kc][0], sx[kc][1], acc, lane);
                    __syncwarp();
                    if (lane == 0) fill_next(st);
                    if (++st == NSTAGE) { st = 0; par ^= 1; }
                }
            }
            if (!alive) break;
            // this warp's partial sums of the real tile columns join the result
            #pragma unroll
            for (int c = 0; c < 2; ++c)
            {
                if (2 * q + c < nrows)
                {
                    float* yr = (c ? outB : outA) + j * 64;
                    #pragma unroll
                    for (int ss = 0; ss < 4; ++ss)
                    {
                        red_add(yr + ss * 16, acc[ss][c] * sd[2 * ss]);
                        red_add(yr + ss * 16 + 8, acc[ss][2 + c] * sd[2 * ss + 1]);
                    }
                }
            }
            #pragma unroll
            for (int ss = 0; ss < 4; ++ss) acc[ss][0] = acc[ss][1] = acc[ss][2] = acc[ss][3] = 0.f;
            if (same_tile)
            {
                ++j;
                #pragma unroll
                for (int k = 0; k < 8; ++k) sd[k] = sdn[k];
            }
            else if (p + 1 < p1)
            {
                j = 0; ++tile;
                enter_tile(tile);
                if (!GROUPED) load_row_scales(j, sd);
            }
        }
    }
    else if (DOWN) { pdl_wait(); pdl_launch_dependents(); }
    __syncthreads();
    TL_MAX(DOWN ? 9 : 1);
    if (DOWN && a.ep.world > 0) ep_tail_combine(a.ep, *a.gen_ptr, a.slot_stride, a.H);
}

}  // namespace

// ---------------------------------------------------------------------------------------------------------------------
// host side
static size_t up256(size_t b) { return (b + 255) / 256 * 256; }

size_t decode_ws_bytes(int H, int I)
{
    size_t b = 256;                                      // status word + padding
    b += up256(sizeof(Route));
    b += up256((size_t) MAXR * H * 2);                   // xf
    b += up256((size_t) MAXR * (H / 32) * 4);            // xscale
    b += up256((size_t) MAXT * 8 * I * 2);               // act
    b += up256((size_t) MAXT * 8 * (I / 32) * 4);        // ascale
    return b;
}

// Optional phase timing: when switched on, every decode call records four events (before prepare, after prepare, after
// gate_up, after down) on the caller's stream into a ring of PROF_RING sets; decode_phase_times() averages the sets recorded
// since profiling was switched on (at most the last PROF_RING calls). Programmatic dependent launch is off meanwhile.
constexpr int PROF_RING = 32;
static bool g_prof = false;
static cudaEvent_t g_ev[PROF_RING][4];
static bool g_ev_made = false;
static unsigned g_prof_calls = 0;

int decode_set_profiling(int on)
{
    if (on && !g_ev_made)
    {
        for (int i = 0; i < PROF_RING * 4; ++i)
            if (cudaEventCreate(&g_ev[i / 4][i % 4]) != cudaSuccess) return fail(HMOE_E_CUDA, "hmoe_set_profiling: cudaEventCreate failed");
        g_ev_made = true;
    }
    if (on && !g_prof) g_prof_calls = 0;
    g_prof = on != 0;
    return HMOE_OK;
}

int decode_phase_times(float* ms3)
{
    if (!g_ev_made || g_prof_calls == 0) return fail(HMOE_E_ARG, "hmoe_decode_phase_times: no call was timed");
    const unsigned n = g_prof_calls < PROF_RING ? g_prof_calls : PROF_RING;
    ms3[0] = ms3[1] = ms3[2] = 0.f;
    for (unsigned s = 0; s < n; ++s)
    {
        if (cudaEventSynchronize(g_ev[s][3]) != cudaSuccess) return fail(HMOE_E_CUDA, "hmoe_decode_phase_times: no timed call");
        for (int i = 0; i < 3; ++i)
        {
            float ms = 0.f;
            if (cudaEventElapsedTime(&ms, g_ev[s][i], g_ev[s][i + 1]) != cudaSuccess) return fail(HMOE_E_CUDA, "hmoe_decode_phase_times: elapsed");
            ms3[i] += ms / n;
        }
    }
    return HMOE_OK;
}

template <typename Kern>
static void launch_dependent(Kern kern, int grid, const DecodeArgs& a, cudaStream_t st)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(NTHREADS); cfg.dynamicSmemBytes = StreamSmem::total; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = g_prof ? 0 : 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, kern, a);
}

template <bool G, bool Q, int KC>
static void launch_stream_gate_up(int grid, const DecodeArgs& a, cudaStream_t st)
{
    static DeviceOnce once;
    if (once.first()) cudaFuncSetAttribute(decode_stream_kernel<G, Q, false, KC>, cudaFuncAttributeMaxDynamicSharedMemorySize, StreamSmem::total);
    launch_dependent(decode_stream_kernel<G, Q, false, KC>, grid, a, st);
}

template <bool G, bool Q>
static void launch_pair(int grid, const DecodeArgs& a, int R, cudaStream_t st)
{
    cudaEvent_t* ev = g_ev[g_prof_calls % PROF_RING];
    if (g_prof) cudaEventRecord(ev[1], st);
    static DeviceOnce once;
    if (once.first())
    {
        cudaFuncSetAttribute(decode_gate_up_kernel<G, Q>, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemLayout::total);
        cudaFuncSetAttribute(decode_down_kernel<G, Q>, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemLayout::total);
        cudaFuncSetAttribute(decode_stream_kernel<G, Q, true, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, StreamSmem::total);
    }
    const bool resident = a.I <= 2048 && a.H <= 6144;      // the activation fragments of a tile fit in registers
    if (!resident) decode_gate_up_kernel<G, Q><<<grid, NTHREADS, SmemLayout::total, st>>>(a);
    else if (a.H <= 2048) launch_stream_gate_up<G, Q, 1>(grid, a, st);
    else if (a.H <= 4096) launch_stream_gate_up<G, Q, 2>(grid, a, st);
    else launch_stream_gate_up<G, Q, 3>(grid, a, st);
    if (g_prof) cudaEventRecord(ev[2], st);
    if (resident) launch_dependent(decode_stream_kernel<G, Q, true, 1>, grid, a, st);
    else decode_down_kernel<G, Q><<<grid, NTHREADS, SmemLayout::total, st>>>(a, R);
    if (g_prof) { cudaEventRecord(ev[3], st); ++g_prof_calls; }
}

// The arguments of the set-up step for a call with these parameters (for the router's launch, which can do the step itself).
int decode_prep_args(const hmoe_layer* L, const void* x, int x_dtype, int R, int lo, int n_local, int act_quant, void* ws, size_t ws_bytes,
                     int sh_mod, int sh_rem, unsigned* gen_ptr, PrepArgs* pa)
{
    const int H = L->H, I = L->I;
    if (R < 1 || R > MAXR || H % 128 || I % 128 || H < 128 || I < 128 || !ws || ws_bytes < decode_ws_bytes(H, I)) return fail(HMOE_E_ARG, "hmoe_router_decode: shapes or workspace");
    if (x_dtype != HMOE_F16 && x_dtype != HMOE_BF16) return fail(HMOE_E_ARG, "hmoe_router_decode: x must be fp16 or bf16");
    const int sms = device_sms();
    if (sms <= 0) return fail(HMOE_E_CUDA, "hmoe_router_decode: no current CUDA device");
    char* w = (char*) ws;
    pa->status = (unsigned*) w; w += 256;
    pa->route = (Route*) w; w += up256(sizeof(Route));
    pa->xf = (__half*) w; w += up256((size_t) MAXR * H * 2);
    pa->xscale = (float*) w; w += up256((size_t) MAXR * (H / 32) * 4);
    pa->gzero = (float4*) w;
    pa->gzero_n = (I <= 2048 && H <= 6144) ? (L->topk + 1) * 2 * I / 4 : 0;
    const bool sh8 = L->shared_format == 1 && L->sh_gate_w != nullptr;
    pa->x = x; pa->x_kind = x_dtype == HMOE_BF16 ? 1 : 0; pa->act_quant = act_quant;
    pa->lo = lo; pa->n_local = n_local; pa->has_shared = L->sh_gate_w != nullptr && !sh8; pa->sh_mod = sh_mod; pa->sh_rem = sh_rem;
    pa->gen_bump = gen_ptr; pa->I = I; pa->nblocks = sms < MAXB ? sms : MAXB;
    return HMOE_OK;
}

int decode_launch(const hmoe_layer* L, const void* x, int x_dtype, const int64_t* sel, const void* rw, int R, int lo, int n_local,
                  int act_quant, float* y, void* ws, size_t ws_bytes, cudaStream_t st, int sh_mod, int sh_rem, unsigned* gen_ptr, size_t slot_stride,
                  bool prepared, const EpCombineArgs* epc)
{
    if (sh_mod < 1 || sh_rem < 0 || sh_rem >= sh_mod) return fail(HMOE_E_ARG, "hmoe_decode: shared-row split must satisfy 0 <= rem < mod");
    const int H = L->H, I = L->I;
    if (R < 1 || R > MAXR) return fail(HMOE_E_ARG, "hmoe_decode: rows must be 1..16");
    if (L->topk < 1 || L->topk > TOPK_MAX) return fail(HMOE_E_ARG, "hmoe_decode: topk must be 1..8");
    if (H % 128 || I % 128 || H < 128 || I < 128) return fail(HMOE_E_ARG, "hmoe_decode: H and I must be multiples of 128");
    if (n_local < 0 || n_local > 256) return fail(HMOE_E_ARG, "hmoe_decode: at most 256 local experts");
    if (!(L->group == 0 && L->scale_dtype == HMOE_F32) && !(L->group == 128 && L->scale_dtype == HMOE_BF16))
        return fail(HMOE_E_ARG, "hmoe_decode: scales must be fp32 per row (group 0) or bf16 per 128 columns");
    if (x_dtype != HMOE_F16 && x_dtype != HMOE_BF16 && x_dtype != HMOE_F16_FRAG) return fail(HMOE_E_ARG, "hmoe_decode: x must be fp16 or bf16");
    if (ws_bytes < decode_ws_bytes(H, I)) return fail(HMOE_E_WS, "hmoe_decode: workspace too small");
    if (!x || !sel || !rw || !y || !ws) return fail(HMOE_E_ARG, "hmoe_decode: null pointer");
    const int g_sms = device_sms();
    if (g_sms <= 0) return fail(HMOE_E_CUDA, "hmoe_decode: no current CUDA device");
    char* w = (char*) ws;
    unsigned* status = (unsigned*) w; w += 256;
    Route* route = (Route*) w; w += up256(sizeof(Route));
    __half* xf = (__half*) w; w += up256((size_t) MAXR * H * 2);
    float* xscale = (float*) w; w += up256((size_t) MAXR * (H / 32) * 4);
    __half* act = (__half*) w; w += up256((size_t) MAXT * 8 * I * 2);
    float* ascale = (float*) w;
    const bool sh8 = L->shared_format == 1 && L->sh_gate_w != nullptr;       // the reference's int8 shared expert: its own kernels
    if (sh8 && !(I <= 2048 && H <= 6144)) return fail(HMOE_E_UNSUPPORTED, "hmoe_decode: the int8 shared expert needs H <= 6144 and I <= 2048");
    // its kernels read the prepared rows as values; in the int8 activation mode those hold codes with their scales apart
    if (sh8 && act_quant) return fail(HMOE_E_UNSUPPORTED, "hmoe_decode: the int8 shared expert is not available in the int8 activation mode (hmoe_prefill serves it)");
    const int has_shared = L->sh_gate_w != nullptr && !sh8;
    if (g_prof) cudaEventRecord(g_ev[g_prof_calls % PROF_RING][0], st);
    // prepared: the router's launch has done the set-up step (hmoe_router_decode)
    if (!prepared) decode_prepare_kernel<<<R + 1, 256, 0, st>>>(x, x_dtype == HMOE_BF16 ? 1 : (x_dtype == HMOE_F16_FRAG ? 2 : 0), sel, (const __half*) rw, R, H, L->topk, lo, n_local, has_shared,
                                                 act_quant, xf, xscale, route, sh_mod, sh_rem, gen_ptr,
                                                 (float4*) act, (I <= 2048 && H <= 6144) ? (L->topk + 1) * 2 * I / 4 : 0, I, g_sms < MAXB ? g_sms : MAXB);
    if (sh8)
    {
        // its gate / up sums go to the rows of the per-pick buffer behind the routed picks (cleared by the prepare kernel with the rest)
        const int rc = shared_i8_launch(L, R, sh_mod, sh_rem, xf, (float*) act + (size_t) R * L->topk * 2 * I, y, gen_ptr, slot_stride,
                                        g_sms < MAXB ? g_sms : MAXB, st);
        if (rc) return rc;
    }
    DecodeArgs a;
    a.H = H; a.I = I;
    a.gate_w = L->gate_w; a.up_w = L->up_w; a.down_w = L->down_w; a.gate_s = L->gate_s; a.up_s = L->up_s; a.down_s = L->down_s;
    a.sh_gw = sh8 ? nullptr : L->sh_gate_w; a.sh_uw = sh8 ? nullptr : L->sh_up_w; a.sh_dw = sh8 ? nullptr : L->sh_down_w;
    a.sh_gs = sh8 ? nullptr : L->sh_gate_s; a.sh_us = sh8 ? nullptr : L->sh_up_s; a.sh_ds = sh8 ? nullptr : L->sh_down_s;
    a.route = route; a.xf = xf; a.xscale = xscale; a.act = act; a.ascale = ascale; a.G = (float*) act; a.y = y; a.status = status;
    a.gen_ptr = gen_ptr; a.slot_stride = slot_stride;
    a.ep = EpTail();
    if (epc)
    {
        if (!gen_ptr || !(I <= 2048 && H <= 6144)) return fail(HMOE_E_UNSUPPORTED, "hmoe_decode_ep_combine: needs the step counter and H <= 6144, I <= 2048");
        if (epc->world < 1 || epc->world > 8 || epc->rank < 0 || epc->rank >= epc->world || !epc->f || !epc->slots || !epc->flags || !epc->status || H % 4 ||
            (size_t) R * H > slot_stride)
            return fail(HMOE_E_ARG, "hmoe_decode_ep_combine: world 1..8, buffers, rows * H <= slot_floats");
        a.ep.rank = epc->rank; a.ep.world = epc->world; a.ep.own_rows = epc->own_rows; a.ep.n = R * H; a.ep.f = epc->f;
        a.ep.done = status + 4; a.ep.status = epc->status;
        for (int p = 0; p < 8; ++p) { a.ep.slots[p] = p < epc->world ? (float*) epc->slots[p] : nullptr; a.ep.flags[p] = p < epc->world ? (unsigned*) epc->flags[p] : nullptr; }
    }
    const int grid = g_sms < MAXB ? g_sms : MAXB;
    const int v = (L->group ? 2 : 0) + (act_quant ? 1 : 0);
    if (v == 0) launch_pair<false, false>(grid, a, R, st);
    else if (v == 1) launch_pair<false, true>(grid, a, R, st);
    else if (v == 2) launch_pair<true, false>(grid, a, R, st);
    else launch_pair<true, true>(grid, a, R, st);
    count_launches(prepared ? 2 : 3);
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return fail(HMOE_E_CUDA, cudaGetErrorString(err));
    return HMOE_OK;
}

// ---------------------------------------------------------------------------------------------------------------------
// Short prefill (1 .. SHORT_MAXR rows): set-up kernel + the two streaming kernels over one tile list for the whole call.
size_t short_ws_bytes(int R, int H, int I, int topk)
{
    size_t b = 256;                                      // status word + padding
    b += up256(sizeof(RouteShort));
    b += up256((size_t) R * H * 2);                      // xf
    b += up256((size_t) R * (H / 32) * 4);               // xscale
    b += up256((size_t) R * (topk + 1) * 2 * I * 4);     // per-pick gate / up sums
    return b;
}

template <bool G, bool Q, int KC>
static void launch_short_gate_up(int grid, const DecodeArgs& a, cudaStream_t st)
{
    static DeviceOnce once;
    if (once.first()) cudaFuncSetAttribute(decode_stream_kernel<G, Q, false, KC, RouteShort>, cudaFuncAttributeMaxDynamicSharedMemorySize, StreamSmem::total);
    launch_dependent(decode_stream_kernel<G, Q, false, KC, RouteShort>, grid, a, st);
}

template <bool G, bool Q>
static void launch_short_pair(int grid, const DecodeArgs& a, cudaStream_t st)
{
    static DeviceOnce once;
    if (once.first()) cudaFuncSetAttribute(decode_stream_kernel<G, Q, true, 1, RouteShort>, cudaFuncAttributeMaxDynamicSharedMemorySize, StreamSmem::total);
    if (a.H <= 2048) launch_short_gate_up<G, Q, 1>(grid, a, st);
    else if (a.H <= 4096) launch_short_gate_up<G, Q, 2>(grid, a, st);
    else launch_short_gate_up<G, Q, 3>(grid, a, st);
    launch_dependent(decode_stream_kernel<G, Q, true, 1, RouteShort>, grid, a, st);
}

int short_launch(const hmoe_layer* L, const void* x, int x_dtype, const int64_t* sel, const void* rw, int R, int lo, int n_local,
                 int act_quant, float* y, void* ws, size_t ws_bytes, cudaStream_t st, int shared_row0, int shared_rows)
{
    const int H = L->H, I = L->I;
    if (shared_rows < 0) { shared_row0 = 0; shared_rows = R; }
    if (shared_row0 < 0 || shared_row0 + shared_rows > R) return fail(HMOE_E_ARG, "hmoe_short_prefill: the shared expert's rows must lie inside the call's rows");
    if (R < 1 || R > SHORT_MAXR) return fail(HMOE_E_ARG, "hmoe_short_prefill: rows must be 1..640");
    if (L->topk < 1 || L->topk > TOPK_MAX) return fail(HMOE_E_ARG, "hmoe_short_prefill: topk must be 1..8");
    if (H % 128 || I % 128 || H < 128 || I < 128) return fail(HMOE_E_ARG, "hmoe_short_prefill: H and I must be multiples of 128");
    if (!(I <= 2048 && H <= 6144)) return fail(HMOE_E_UNSUPPORTED, "hmoe_short_prefill: needs H <= 6144 and I <= 2048");
    const bool sh8 = L->shared_format == 1 && L->sh_gate_w != nullptr;       // the reference's int8 shared expert: its own kernels, 16 rows at a time
    if (sh8 && act_quant) return fail(HMOE_E_UNSUPPORTED, "hmoe_short_prefill: the int8 shared expert is not available in the int8 activation mode (hmoe_prefill serves it)");
    if (n_local < 0 || n_local > 256) return fail(HMOE_E_ARG, "hmoe_short_prefill: at most 256 local experts");
    if (!(L->group == 0 && L->scale_dtype == HMOE_F32) && !(L->group == 128 && L->scale_dtype == HMOE_BF16))
        return fail(HMOE_E_ARG, "hmoe_short_prefill: scales must be fp32 per row (group 0) or bf16 per 128 columns");
    if (x_dtype != HMOE_F16 && x_dtype != HMOE_BF16) return fail(HMOE_E_ARG, "hmoe_short_prefill: x must be fp16 or bf16");
    if (!x || !sel || !rw || !y || !ws) return fail(HMOE_E_ARG, "hmoe_short_prefill: null pointer");
    if (ws_bytes < short_ws_bytes(R, H, I, L->topk)) return fail(HMOE_E_WS, "hmoe_short_prefill: workspace too small");
    const int g_sms = device_sms();
    if (g_sms <= 0) return fail(HMOE_E_CUDA, "hmoe_short_prefill: no current CUDA device");
    char* w = (char*) ws;
    unsigned* status = (unsigned*) w; w += 256;
    RouteShort* route = (RouteShort*) w; w += up256(sizeof(RouteShort));
    __half* xf = (__half*) w; w += up256((size_t) R * H * 2);
    float* xscale = (float*) w; w += up256((size_t) R * (H / 32) * 4);
    float* G = (float*) w;
    const int has_shared = L->sh_gate_w != nullptr && shared_rows > 0 && !sh8;
    const int grid = g_sms < MAXB ? g_sms : MAXB;
    short_prepare_kernel<<<R + 1, SHORT_THREADS, 0, st>>>(x, x_dtype == HMOE_BF16 ? 1 : 0, sel, (const __half*) rw, R, H, L->topk, lo, n_local, has_shared,
                                                          act_quant, xf, xscale, route, shared_row0, shared_rows, (float4*) G, (L->topk + 1) * 2 * I / 4, I, grid);
    if (sh8)
    {
        // The shared expert's rows in groups of sixteen through the decode path's pair of int8 kernels; a group's gate / up sums go to
        // sixteen rows of the per-pick buffer behind the routed picks (cleared by the set-up kernel with the rest).
        for (int c = 0; c < shared_rows; c += MAXR)
        {
            const int n = shared_rows - c < MAXR ? shared_rows - c : MAXR, r0 = shared_row0 + c;
            const int rc = shared_i8_launch(L, n, 1, 0, xf + (size_t) r0 * H, G + ((size_t) R * L->topk + c) * 2 * I, y + (size_t) r0 * H, nullptr, 0, grid, st);
            if (rc) return rc;
        }
    }
    DecodeArgs a;
    a.H = H; a.I = I;
    a.gate_w = L->gate_w; a.up_w = L->up_w; a.down_w = L->down_w; a.gate_s = L->gate_s; a.up_s = L->up_s; a.down_s = L->down_s;
    a.sh_gw = sh8 ? nullptr : L->sh_gate_w; a.sh_uw = sh8 ? nullptr : L->sh_up_w; a.sh_dw = sh8 ? nullptr : L->sh_down_w;
    a.sh_gs = sh8 ? nullptr : L->sh_gate_s; a.sh_us = sh8 ? nullptr : L->sh_up_s; a.sh_ds = sh8 ? nullptr : L->sh_down_s;
    a.route = reinterpret_cast<const Route*>(route); a.xf = xf; a.xscale = xscale; a.act = nullptr; a.ascale = nullptr; a.G = G; a.y = y; a.status = status;
    a.gen_ptr = nullptr; a.slot_stride = 0;
    a.ep = EpTail();
    const int v = (L->group ? 2 : 0) + (act_quant ? 1 : 0);
    if (v == 0) launch_short_pair<false, false>(grid, a, st);
    else if (v == 1) launch_short_pair<false, true>(grid, a, st);
    else if (v == 2) launch_short_pair<true, false>(grid, a, st);
    else launch_short_pair<true, true>(grid, a, st);
    count_launches(3);
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return fail(HMOE_E_CUDA, cudaGetErrorString(err));
    return HMOE_OK;
}

}  // namespace hmoe

// ---------------------------------------------------------------------------------------------------------------------
// Decode with built-in scratch, for hosts that must not allocate.
//
// Some embedders of this library hand out device memory from one arena that is carved up once at start-up (an inference
// server with a fixed memory plan, a plugin running inside another framework's allocator, a real-time loop where a
// cudaMalloc would stall every stream of the process). For them the 4.6 MB workspace of hmoe_decode is one more buffer to
// plan. This variant needs none: its workspace is the array below, which is part of the library image, so every GPU that
// loads the library carries these 5 MiB from load to exit whether or not the entry point is ever called.
//
// The array's name is only meaningful in device code. On the host it is a stand-in symbol, not an address a kernel could
// use, so the device address is looked up with cudaGetSymbolAddress, once per device, with that device current, the first
// time the entry point runs there. That look-up is a set-up step: make the first call on each device outside any stream
// capture. Later calls only launch work.
//
// All calls on one device share the array and it keeps whatever the previous call left. The only word that has to start
// from zero, the status word, is cleared on the caller's stream at the start of every call; everything else is rewritten
// by the call's own prepare and gate_up kernels before it is read. Two calls whose kernels overlap on the GPU (different
// streams, or graph branches without an edge between them) would overwrite each other's intermediate results: keep the
// calls of one device ordered.
namespace hmoe {
namespace {
constexpr size_t STATIC_WS_BYTES = 5u << 20;
static __device__ __align__(256) unsigned char g_decode_scratch[STATIC_WS_BYTES];
static void* g_scratch_addr[MAX_DEVICES] = {};
}  // namespace
}  // namespace hmoe

extern "C" int hmoe_decode_noalloc(const hmoe_layer* layer, const void* x, int x_dtype, const int64_t* sel, const void* rw, int R,
                                   int lo, int n_local, int act_quant, float* y, uint32_t* status_dev, void* stream)
{
    using namespace hmoe;
    if (!layer) return fail(HMOE_E_ARG, "hmoe_decode_noalloc: null layer");
    const size_t need = decode_ws_bytes(layer->H, layer->I);
    if (layer->H <= 0 || layer->I <= 0 || need > STATIC_WS_BYTES)
        return fail(HMOE_E_WS, "hmoe_decode_noalloc: H / I exceed the built-in scratch (5 MiB: up to H = 6144 with I = 2048); "
                               "use hmoe_decode with a caller-provided workspace");
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES)
        return fail(HMOE_E_CUDA, "hmoe_decode_noalloc: no current CUDA device (or device index >= 64)");
    if (!g_scratch_addr[dev])
    {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_decode_scratch);
        if (e != cudaSuccess || !p) return fail(HMOE_E_CUDA, cudaGetErrorString(e));
        g_scratch_addr[dev] = p;
    }
    void* ws = g_scratch_addr[dev];
    cudaStream_t st = (cudaStream_t) stream;
    if (cudaMemsetAsync(ws, 0, 256, st) != cudaSuccess) return fail(HMOE_E_CUDA, "hmoe_decode_noalloc: clearing the status word failed");
    const int rc = decode_launch(layer, x, x_dtype, sel, rw, R, lo, n_local, act_quant, y, ws, STATIC_WS_BYTES, st);
    if (rc != HMOE_OK) return rc;
    if (status_dev && cudaMemcpyAsync(status_dev, ws, 4, cudaMemcpyDeviceToDevice, st) != cudaSuccess)
        return fail(HMOE_E_CUDA, "hmoe_decode_noalloc: copying the status word failed");
    return HMOE_OK;
}

#ifdef HMOE_PROBE_TIMELINE
using namespace hmoe;
TL_READER(hmoe_tl_decode)
#endif

// Prefill path of the MoE expert layer (hundreds to tens of thousands of rows), sm_100a: token permutation on the device
// and two grouped GEMMs on the tcgen05 tensor cores with the int4 weights dequantised on the way into shared memory.
//
// Replaces, behind the same operator surface (packed int4 experts in the reference's fragment order, (sel, rw) routing, fp32
// output added into `out`):
//   * the host-side permutation of runtime/tier/tier_split.py:404-412,433-455 (stable argsort by expert id, bincount with a
//     host sync, numpy row blocks from runtime/tier/rtx_split.py:236-255 copied to the device per group) by three small
//     kernels with no host synchronisation: histogram per 1024-pick chunk, scan + balanced row-block table, stable scatter;
//   * gather_kernel / p4t_gu_kernel / p4t_gemm_kernel of runtime/tier/moe4/moe4t.cu:113-433 by the kernels below.
//
// GEMM orientation: D[channel][pick] = W[channel][k] . X[pick][k]: the weights are the M = 128 operand, the picks of one
// row block (<= 256, one expert) the N operand, fp32 accumulators in tensor memory. Per 64-column stage:
//   warps 0-15 read the packed codes of the tile straight from global memory (16 bytes per lane, the stored fragment order),
//              turn them into fp16 (times the bf16 group scale in the group format) and store them as a K-major,
//              128-byte-swizzled operand tile (16-byte stores, conflict free); they do nothing else and run ahead of the MMAs
//              from tile to tile as far as the ring allows;
//   warp 16    one thread loads the row block's input tile (picks x 64 columns) as 2-D TMA boxes of 64 rows, as many as the block
//              has picks (128-byte swizzle, rows beyond the array zero-filled);
//   warp 17    one thread issues tcgen05.mma (M 128, N = picks rounded up to 16, K 16) four times per matrix and commits the
//              stage back to the producers;
//   warps 18-21 (down) / 18-25 (gate_up) read the finished sums out of tensor memory (one quarter of the lanes = 32 channels each;
//              gate_up: two warps per quarter, half the columns each).
// gate_up keeps two accumulators (gate, up: 2 x 256 columns) over the same input tile and its read-out writes
// act = SiLU(g) * u * routing weight in fp16; down adds scale * sum into out[token] with coalesced fp32 reductions and keeps two
// accumulator sets, so a tile's read-out runs under the next tile's MMAs. (Measured on the benchmark with parts of the kernel
// switched off: the MMA / TMA pipeline alone needs 4.5 ms of a 7.7 ms step, the dequantisation 1.5 ms and the read-outs 1.7 ms
// when the same warps do both in turn, as an earlier version did; hence the separate warps.)
// Blocks are persistent (one per SM) over (row block, channel tile) items, channel tile fastest, so the blocks working at
// the same time share one input tile and one expert's weights through L2.
// Every wait is bounded (see mbar_wait); tensor memory is released by the warp that allocated it on every path.
#include <cuda.h>
#include <type_traits>
#include "hmoe_common.cuh"
#include "hmoe_internal.h"

namespace hmoe {
namespace {

// Diagnostic build (-DHMOE_PROBE_WAITS): every role adds up the cycles it spends in each of its waits (in registers, one atomic
// per thread at the end of the kernel); hmoe_probe_read() returns the sums. 32 counters per kernel: 0 / 1 / 2 MMA thread waiting
// for the weights / the inputs / a free accumulator set, 4 and 10 dequantising warps 0 and 15 waiting for a ring slot, 9 warp 0's
// stores + fence + arrive, 6 TMA thread waiting for a slot, 7 / 8 first read-out warp waiting for a tile / reading it out, 15
// the block's lifetime. Not part of the normal build.
#ifdef HMOE_PROBE_WAITS
__device__ unsigned long long g_probe[64];
#define PROBE_T0() const long long pt0_ = clock64()
#define PROBE_ADD(i) pacc_[i] += (unsigned long long) (clock64() - pt0_)
#define PROBE_ON(c) (c)
#else
#define PROBE_T0()
#define PROBE_ADD(i)
#define PROBE_ON(c) false
#endif
constexpr int TM = 128, TN = 256, TK = 64;
constexpr int TB = 64;                          // rows per TMA box of the input tile
constexpr int NDQ = 16;                         // dequantising warps
// read-out warps: one per quarter of the tensor-memory lanes in down (whose read-out runs under the next tile's MMAs), two per
// quarter in gate_up (whose single accumulator set keeps the tensor core waiting until the read-out is done: half the columns each)
__host__ __device__ constexpr int nepi(int nmat) { return nmat == 2 ? 8 : 4; }
__host__ __device__ constexpr int pf_threads(int nmat) { return (NDQ + 2 + nepi(nmat)) * 32; }      // warp NDQ: TMA, warp NDQ + 1: MMA, warps NDQ + 2 ..: read-out
constexpr int CHUNK = 1024;                     // picks per permutation block (one warp)

// ---------------------------------------------------------------------------------------------------------------------
// permutation
struct Plan
{
    int total;          // routed local picks + shared rows
    int nrb;            // row blocks
    int pad[2];
};

// per 1024-pick chunk: how many picks of each local expert
__global__ void __launch_bounds__(32) permute_hist_kernel(const int64_t* __restrict__ sel, int P, int lo, int n_local, int* __restrict__ block_hist)
{
    __shared__ int hist[256];
    const int lane = threadIdx.x, base = blockIdx.x * CHUNK;
    for (int e = lane; e < n_local; e += 32) hist[e] = 0;
    __syncwarp();
    for (int i = base + lane; i < base + CHUNK && i < P; i += 32)
    {
        const int64_t e = sel[i] - lo;
        if (e >= 0 && e < n_local) atomicAdd(&hist[(int) e], 1);
    }
    __syncwarp();
    for (int e = lane; e < n_local; e += 32) block_hist[(size_t) blockIdx.x * n_local + e] = hist[e];
}

// one block: chunk offsets per expert, expert offsets, the shared expert's segment, balanced row blocks
// (runtime/tier/rtx_split.py:236-255 with one pick group: experts without picks emit nothing, an expert's blocks get
// near-equal sizes when `balance`, {expert, first pick, picks, 0})
__global__ void __launch_bounds__(256) permute_scan_kernel(int* __restrict__ block_hist, int nblocks, int n_local, int shared_rows, int bm,
                                                          int balance, int* __restrict__ counts, int* __restrict__ offs, int* __restrict__ rbt,
                                                          Plan* __restrict__ plan)
{
    __shared__ int cnt[257], off[258], rb0[258];
    const int t = threadIdx.x;
    const int ne = n_local + (shared_rows > 0 ? 1 : 0);
    for (int e = t; e < n_local; e += blockDim.x)
    {
        int run = 0;
        for (int b = 0; b < nblocks; ++b) { const int v = block_hist[(size_t) b * n_local + e]; block_hist[(size_t) b * n_local + e] = run; run += v; }
        cnt[e] = run;
    }
    if (t == 0 && shared_rows > 0) cnt[n_local] = shared_rows;
    __syncthreads();
    if (t == 0)
    {
        int o = 0, r = 0;
        for (int e = 0; e < ne; ++e) { off[e] = o; rb0[e] = r; o += cnt[e]; r += (cnt[e] + bm - 1) / bm; }
        off[ne] = o; rb0[ne] = r;
        plan->total = o; plan->nrb = r; plan->pad[0] = plan->pad[1] = 0;
    }
    __syncthreads();
    for (int e = t; e <= ne; e += blockDim.x) { offs[e] = off[e]; if (e < ne) counts[e] = cnt[e]; }
    for (int e = t; e < ne; e += blockDim.x)
    {
        const int c = cnt[e], nb = (c + bm - 1) / bm;
        for (int k = 0; k < nb; ++k)
        {
            int rows, start;
            if (balance) { const int base = c / nb, extra = c % nb; rows = base + (k < extra ? 1 : 0); start = k * base + (k < extra ? k : extra); }
            else { rows = c - bm * k < bm ? c - bm * k : bm; start = bm * k; }
            int* r = rbt + 4 * (rb0[e] + k);
            r[0] = e; r[1] = off[e] + start; r[2] = rows; r[3] = 0;
        }
    }
}

// stable scatter: pick i goes to offs[e] + (picks of e in earlier chunks) + (picks of e earlier in this chunk)
__global__ void __launch_bounds__(32) permute_scatter_kernel(const int64_t* __restrict__ sel, const __half* __restrict__ rw, int P, int topk,
    int lo, int n_local, int shared_rows, int shared_row0, const int* __restrict__ block_hist, const int* __restrict__ offs, int nblocks,
    int* __restrict__ order, int* __restrict__ tok, int* __restrict__ eid, float* __restrict__ wt)
{
    const int lane = threadIdx.x;
    if ((int) blockIdx.x >= nblocks)
    {
        // the shared expert's rows: every row once, in order, weight 1
        const int base = ((int) blockIdx.x - nblocks) * CHUNK, o = offs[n_local];
        for (int r = base + lane; r < base + CHUNK && r < shared_rows; r += 32) { tok[o + r] = shared_row0 + r; eid[o + r] = n_local; wt[o + r] = 1.f; if (order) order[o + r] = -1; }
        return;
    }
    __shared__ int seen[256];
    for (int e = lane; e < n_local; e += 32) seen[e] = 0;
    __syncwarp();
    const int base = blockIdx.x * CHUNK;
    for (int i0 = base; i0 < base + CHUNK && i0 < P; i0 += 32)
    {
        const int i = i0 + lane;
        int e = -1;
        if (i < P) { const int64_t v = sel[i] - lo; if (v >= 0 && v < n_local) e = (int) v; }
        const unsigned same = __match_any_sync(0xffffffffu, e);
        if (e >= 0)
        {
            const int rank = __popc(same & ((1u << lane) - 1u));
            const int pos = offs[e] + block_hist[(size_t) blockIdx.x * n_local + e] + seen[e] + rank;
            if (order) order[pos] = i;
            tok[pos] = i / topk; eid[pos] = e; wt[pos] = __half2float(rw[i]);
        }
        __syncwarp();
        if (e >= 0 && (same >> lane) == 1u) seen[e] += __popc(same);      // the highest lane of each group updates the count
        __syncwarp();
    }
}

// xg[pos][H] = fp16(x[tok[pos]]), optionally after the CPU engine's int8 round trip (runtime/tier/cpuband.cpp:106-111)
__global__ void __launch_bounds__(192) gather_kernel(const void* __restrict__ x, int x_bf16, const int* __restrict__ tok, const Plan* __restrict__ plan,
                                                     int H, int act_quant, __half* __restrict__ xg)
{
    const int pos = blockIdx.x;
    if (pos >= plan->total) return;
    const int r = tok[pos];
    for (int gi = threadIdx.x; gi < H / 32; gi += blockDim.x)
    {
        float v[32];
        if (x_bf16)
        {
            const uint4* p = (const uint4*) ((const uint16_t*) x + (size_t) r * H + gi * 32);
            #pragma unroll
            for (int j = 0; j < 4; ++j)
            {
                const uint4 u = p[j]; const uint32_t w[4] = {u.x, u.y, u.z, u.w};
                #pragma unroll
                for (int k = 0; k < 4; ++k) { v[j * 8 + 2 * k] = __uint_as_float(w[k] << 16); v[j * 8 + 2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u); }
            }
        }
        else
        {
            const uint4* p = (const uint4*) ((const __half*) x + (size_t) r * H + gi * 32);
            #pragma unroll
            for (int j = 0; j < 4; ++j)
            {
                const uint4 u = p[j]; const uint32_t w[4] = {u.x, u.y, u.z, u.w};
                #pragma unroll
                for (int k = 0; k < 4; ++k) { const float2 f = __half22float2(*(const __half2*) &w[k]); v[j * 8 + 2 * k] = f.x; v[j * 8 + 2 * k + 1] = f.y; }
            }
        }
        if (act_quant)
        {
            float m = 0.f;
            #pragma unroll
            for (int k = 0; k < 32; ++k) m = fmaxf(m, fabsf(v[k]));
            const float s = m > 0.f ? __fdiv_rn(m, 127.f) : 1.f, inv = __fdiv_rn(1.f, s);
            #pragma unroll
            for (int k = 0; k < 32; ++k) v[k] = __fmul_rn((float) __float2int_rn(__fmul_rn(v[k], inv)), s);
        }
        const size_t rowlen = act_quant ? 2 * (size_t) H : (size_t) H;       // int8 mode: [hi | lo] halves, code x scale kept to ~22 bits
        // The 64 columns of a block are stored in the order the weight tiles use (operand_pos): the thread's 32 columns (16-column
        // steps 2j, 2j + 1 of the block) become, for each q, eight consecutive values = one 16-byte store.
        const int kb = gi >> 1, j8 = (gi & 1) * 8;
        #pragma unroll
        for (int q = 0; q < 4; ++q)
        {
            uint32_t w[4], wl[4];
            #pragma unroll
            for (int i = 0; i < 4; ++i)
            {
                const int c = (i >> 1) * 16 + (i & 1) * 8 + 2 * q;           // step (i / 2), half (i % 2), columns 2q, 2q + 1
                const __half2 h = __floats2half2_rn(v[c], v[c + 1]);
                w[i] = *(const uint32_t*) &h;
                const float2 f = __half22float2(h);
                const __half2 l = __floats2half2_rn(v[c] - f.x, v[c + 1] - f.y);
                wl[i] = *(const uint32_t*) &l;
            }
            *(uint4*) (xg + (size_t) pos * rowlen + kb * 64 + q * 16 + j8) = make_uint4(w[0], w[1], w[2], w[3]);
            if (act_quant) *(uint4*) (xg + (size_t) pos * rowlen + H + kb * 64 + q * 16 + j8) = make_uint4(wl[0], wl[1], wl[2], wl[3]);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// tcgen05 helpers
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// shared-memory operand descriptor: K-major tile, 128-byte swizzle, rows of 128 bytes, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr)
{
    return (uint64_t) ((addr & 0x3FFFFu) >> 4) | ((uint64_t) 1 << 16) | ((uint64_t) (1024 >> 4) << 32) | ((uint64_t) 1 << 46) | ((uint64_t) 2 << 61);
}
__device__ __forceinline__ void mma_f16_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r)
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                   "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
                   "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
                   "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]) : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, uint32_t* r)
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63]) : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r)
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                   "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]) : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t* r)
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"((uint64_t) map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void red_add_sys(float* p, float v)
{
    asm volatile("red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(__cvta_generic_to_global(p)), "f"(v) : "memory");
}
__device__ __forceinline__ void sts32(uint32_t addr, uint32_t v) { asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(v) : "memory"); }

struct GemmArgs
{
    int K, N;                 // reduction length and output channels of the matrix (gate_up: K = H, N = I; down: K = I, N = H)
    int grouped;              // bf16 scale per 128 columns (else fp32 per row)
    int act_quant;
    int kfold;                // 1, or 2 in the int8 mode: the inputs are [hi | lo] halves over 2 K columns, the weights are walked twice
    const int64_t* w0; const int64_t* w1;     // pointer tables of the matrix (gate, up) or (down, -)
    const int64_t* s0; const int64_t* s1;     // scale tables
    const void* sh_w0; const void* sh_w1; const void* sh_s0; const void* sh_s1;   // shared expert (expert id n_local)
    int sh_i8;                // the shared expert is in the reference's int8 format (dense GEMV fragment order, fp32 scale per row)
    int n_local;
    const Plan* plan; const int* rbt; const int* tok; const float* wt;
    __half* act;              // gate_up: output [pos][I]
    float* out;               // down: output [R][H], added into
    float* out_peer[8];       // expert parallel, combine over peer memory: row t belongs to rank t / rows_per_rank and is added
    int rows_per_rank;        //   into out_peer[rank][(t % rows_per_rank)][H] (peer pointers over NVLink); 0 = off
    unsigned* status;
};

// Column order of the GEMM operands inside every block of 64 columns. The tensor core only needs both operands to agree on
// which stored position holds which column, so the order is chosen for the weights: a lane (g, q) of the dequantising warps holds,
// of rows g and g + 8, the columns 16 t + 8 h + 2 q + cc (t = 0..3, h, cc = 0..1) of the block, and these go to positions
// 16 q + 4 t + 2 h + cc: the lane's sixteen values of a row are contiguous (32 bytes, two 16-byte stores). The gathered inputs
// and the intermediate activations are written in the same order (gather_kernel, the gate_up read-out).
__host__ __device__ __forceinline__ int operand_pos(int k) { return ((k >> 1) & 3) * 16 + (k >> 4) * 4 + ((k >> 3) & 1) * 2 + (k & 1); }

__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d)
{
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// One 16-row x 64-column strip of packed codes (one 16-byte word per lane) -> 32 fp16 values per lane (a[t] = the four registers
// of 16-column step t, times the group scale), and their store into the K-major 128-byte-swizzled operand tile as four 16-byte
// words (conflict free: the eight lanes of a quarter warp hit eight different 16-byte columns). The two halves are separate
// functions because the conversion is done BEFORE the warp waits for its ring slot: when the slot is released only the four
// stores stand between the release and the MMA thread's wake-up.
__device__ __forceinline__ void convert_strip(const uint4& w, uint32_t s_lo, uint32_t s_hi, bool scaled, uint32_t (&a)[4][4])
{
    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
    #pragma unroll
    for (int t = 0; t < 4; ++t)
    {
        frag_from_codes(ww[t], a[t]);
        if (scaled)
        {
            asm("mul.f16x2 %0, %0, %1;" : "+r"(a[t][0]) : "r"(s_lo)); asm("mul.f16x2 %0, %0, %1;" : "+r"(a[t][2]) : "r"(s_lo));
            asm("mul.f16x2 %0, %0, %1;" : "+r"(a[t][1]) : "r"(s_hi)); asm("mul.f16x2 %0, %0, %1;" : "+r"(a[t][3]) : "r"(s_hi));
        }
    }
}
// row0 = shared address of the lane's row g in the strip's first 8-row group; c0, c1 = byte offsets of its two 16-byte columns
__device__ __forceinline__ void store_strip(uint32_t row0, uint32_t c0, uint32_t c1, const uint32_t (&a)[4][4])
{
    sts128(row0 + c0, a[0][0], a[0][2], a[1][0], a[1][2]);
    sts128(row0 + c1, a[2][0], a[2][2], a[3][0], a[3][2]);
    sts128(row0 + 1024 + c0, a[0][1], a[0][3], a[1][1], a[1][3]);
    sts128(row0 + 1024 + c1, a[2][1], a[2][3], a[3][1], a[3][3]);
}

// bf16 pair (rows g, g + 8 of a strip) -> two fp16x2 broadcast registers
__device__ __forceinline__ void scale_pair(uint32_t bf2, uint32_t& s_lo, uint32_t& s_hi)
{
    const __half2 lo = __float2half2_rn(__uint_as_float(bf2 << 16)), hi = __float2half2_rn(__uint_as_float(bf2 & 0xffff0000u));
    s_lo = *(const uint32_t*) &lo; s_hi = *(const uint32_t*) &hi;
}

template <int NMAT>
struct PfSmem
{
    static constexpr int STAGES = NMAT == 2 ? 3 : 4;
    static constexpr int A_BYTES = TM * TK * 2;             // 16 KB per matrix
    static constexpr int B_BYTES = TN * TK * 2;             // 32 KB
    static constexpr int STAGE = NMAT * A_BYTES + B_BYTES;
    static constexpr int bars = STAGES * STAGE;             // full_a[S], full_b[S], empty[S], done[2], tmem_free[2]
    static constexpr int misc = bars + (3 * STAGES + 4) * 8;
    static constexpr int total = misc + 32 + 1024;          // + slack to align the base to 1024
};

// NMAT = 2: gate and up over one input tile, SiLU epilogue. NMAT = 1: down, scatter-add epilogue.
template <int NMAT>
__global__ void __launch_bounds__(pf_threads(NMAT), 1) prefill_gemm_kernel(const __grid_constant__ CUtensorMap tmap, const GemmArgs a)
{
    using L = PfSmem<NMAT>;
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t sbase = (raw + 1023u) & ~1023u;
    unsigned char* smem = smem_raw + (sbase - raw);
    const uint32_t full_a = sbase + L::bars, full_b = full_a + L::STAGES * 8, empty = full_b + L::STAGES * 8,
                   done = empty + L::STAGES * 8, tmem_free = done + 2 * 8;      // done[NACC], tmem_free[NACC]
    uint32_t* tmem_slot = (uint32_t*) (smem + L::misc);
    volatile int* abort_flag = (volatile int*) (smem + L::misc + 8);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Accumulators in tensor memory: gate + up fill all 512 columns; down needs 256 and keeps two sets, so the MMAs of the
    // next tile run while this tile's sums are read out.
        constexpr int TMEM_COLS = 512, NACC = NMAT == 2 ? 1 : 2;

    if (threadIdx.x == 0)
    {
        for (int i = 0; i < L::STAGES; ++i) { mbar_init(full_a + i * 8, NMAT == 2 ? NDQ : NDQ / 2); mbar_init(full_b + i * 8, 1); mbar_init(empty + i * 8, 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(done + i * 8, 1); mbar_init(tmem_free + i * 8, nepi(NMAT)); }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == NDQ + 1)
    {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    const int KB = a.K / 64, KBT = KB * a.kfold, NCT = a.N / TM;     // KB 64-column blocks of the weights, KBT ring stages per tile
#ifdef HMOE_PROBE_WAITS
    unsigned long long pacc_[16] = {};
#endif
    PROBE_T0();
    const int nitems = a.plan->nrb * NCT;

    if (warp < NDQ)
    {
        // ---- dequantise: one 16-row strip of one 64-row unit per warp and stage. gate_up: 2 matrices x 2 units x 4 strips =
        // 16 strip-blocks per stage, one per warp. down: 8 strip-blocks per stage; warps 0-7 take the even pairs of stages, warps
        // 8-15 the odd ones (in pairs of stages, see below). The packed words are fetched two of the warp's steps ahead. These warps
        // do nothing else: they stream from tile to tile and stop only when the ring is full, so the MMA thread always finds its
        // next stages.
        const int g = lane >> 2, q = lane & 3;
        const int strip = warp & 3, unit = (warp >> 2) & 1, mat = NMAT == 2 ? warp >> 3 : 0;
        const int kb0 = NMAT == 2 ? 0 : warp >> 3, kstep = NMAT == 2 ? 1 : 2;
        // shared address of this lane's row g in slot 0, and its two 16-byte columns under the 128-byte swizzle
        const uint32_t row_off = sbase + mat * L::A_BYTES + (unit * 8 + strip * 2) * 1024 + g * 128;
        const uint32_t c0 = (uint32_t) (((2 * q) ^ g) << 4), c1 = (uint32_t) (((2 * q + 1) ^ g) << 4);
        bool ok = true;
        uint32_t tile_n = 0;
        for (int item = blockIdx.x; item < nitems && ok; item += gridDim.x, ++tile_n)
        {
            if (*abort_flag) { ok = false; break; }
            const int rb = item / NCT, ct = item % NCT, e = a.rbt[4 * rb];
            const void* wp = e < a.n_local ? (const void*) (mat ? a.w1[e] : a.w0[e]) : (mat ? a.sh_w1 : a.sh_w0);
            const void* sp = e < a.n_local ? (const void*) (mat ? a.s1[e] : a.s0[e]) : (mat ? a.sh_s1 : a.sh_s0);
            if (a.sh_i8 && e >= a.n_local)
            {
                // The shared expert in the reference's int8 format (runtime/tier/tier_split.py:495-514): 2 KB units of 64 rows x 32
                // columns, 16 bytes per lane and strip = the fragments of two 16-column steps; a stage takes two units. One ninth
                // of the work at most, so no prefetch queue: the two loads of a stage are issued, converted and stored in turn.
                // Its fp32 row scales are applied by the read-out.
                const char* w8 = (const char*) wp + ((size_t) (2 * ct + unit) * (a.K / 32) * 4 + strip) * 512 + lane * 16;
                const uint32_t it0 = tile_n * (uint32_t) KBT;
                for (int kb = kb0; kb < KBT && ok; kb += kstep)
                {
                    const int kbw = kb >= KB ? kb - KB : kb;
                    const uint4 wa = ldg128_nc(w8 + (size_t) (2 * kbw) * 2048), wb = ldg128_nc(w8 + (size_t) (2 * kbw + 1) * 2048);
                    uint32_t cv[4][4];
                    dec_i8(wa.x, cv[0][0], cv[0][1]); dec_i8(wa.y, cv[0][2], cv[0][3]); dec_i8(wa.z, cv[1][0], cv[1][1]); dec_i8(wa.w, cv[1][2], cv[1][3]);
                    dec_i8(wb.x, cv[2][0], cv[2][1]); dec_i8(wb.y, cv[2][2], cv[2][3]); dec_i8(wb.z, cv[3][0], cv[3][1]); dec_i8(wb.w, cv[3][2], cv[3][3]);
                    const uint32_t gi = it0 + kb, s = gi % L::STAGES;
                    if (gi >= (uint32_t) L::STAGES && !mbar_wait(empty + s * 8, ((gi / L::STAGES) - 1) & 1, abort_flag, a.status)) { ok = false; break; }
                    store_strip(row_off + s * L::STAGE, c0, c1, cv);
                    fence_proxy_async();
                    __syncwarp();
                    mbar_arrive_if(full_a + s * 8, lane == 0);
                }
                continue;
            }
            // One step of a warp = one 128-column scale group = two consecutive ring stages: two 16-byte code words and one scale
            // word per lane. gate_up: every warp takes every pair of stages; down: warps 0-7 the even pairs, warps 8-15 the odd ones.
            const int NPW = KB >> 1, NP = KBT >> 1;                  // pairs in one pass over the weights / in the tile
            const int j0 = NMAT == 2 ? 0 : warp >> 3;
            constexpr int JSTEP = NMAT == 2 ? 1 : 2;
            const char* wbase = (const char*) wp + ((size_t) (2 * ct + unit) * KB * 4 + strip) * 512 + lane * 16;
            const char* sbase_p = (const char*) sp + ((size_t) (2 * ct + unit) * (a.K / 128) * 64 + g * 8 + 2 * strip) * 2;
            // the warp's ring slot and the parity of the slot's current use, stepped from stage to stage (no division per stage)
            const uint32_t gi0 = tile_n * (uint32_t) KBT + 2 * j0;
            uint32_t s = gi0 % L::STAGES, ph = (gi0 / L::STAGES) & 1;
            auto run = [&](auto grouped_tag) {
                constexpr bool GROUPED = decltype(grouped_tag)::value;
                // the code words and scale pairs of the warp's next two steps, in flight while the current step is converted
                uint4 qa[2] = {}, qb[2] = {}; uint32_t qs[2] = {};
                auto fetch = [&](int pj, uint4& wa, uint4& wb, uint32_t& sc) {
                    if (pj >= NP) return;
                    const int jw = pj >= NPW ? pj - NPW : pj;               // second pass over the weights for the lo halves
                    const char* p = wbase + (size_t) jw * 4096;
                    wa = ldg128_nc(p); wb = ldg128_nc(p + 2048);
                    if (GROUPED) sc = __ldg((const uint32_t*) (sbase_p + (size_t) jw * 128));
                };
                // the converted strip into ring slot s (a fresh slot passes at once: its barrier's preceding phase counts as
                // complete), the slot handed to the MMA thread, s stepped
                auto put = [&](const uint32_t (&cv)[4][4]) -> bool {
                    { PROBE_T0(); const bool w_ = mbar_wait(empty + s * 8, ph ^ 1, abort_flag, a.status); if (PROBE_ON(threadIdx.x == 0)) PROBE_ADD(4); if (PROBE_ON(threadIdx.x == 15 * 32)) PROBE_ADD(10); if (!w_) return false; }
                    PROBE_T0();
                    store_strip(row_off + s * L::STAGE, c0, c1, cv);
                    fence_proxy_async();
                    __syncwarp();
                    mbar_arrive_if(full_a + s * 8, lane == 0);
                    if (PROBE_ON(threadIdx.x == 0)) PROBE_ADD(9);
                    if (++s == (uint32_t) L::STAGES) { s = 0; ph ^= 1; }
                    return true;
                };
                fetch(j0, qa[0], qb[0], qs[0]);
                fetch(j0 + JSTEP, qa[1], qb[1], qs[1]);
                uint32_t cv[4][4], s_lo = 0, s_hi = 0;                      // the converted strip of the warp's next stage
                if (GROUPED) scale_pair(qs[0], s_lo, s_hi);
                convert_strip(qa[0], s_lo, s_hi, GROUPED, cv);
                for (int j = j0; j < NP && ok; j += 2 * JSTEP)
                {
                    #pragma unroll
                    for (int u = 0; u < 2; ++u)
                    {
                        const int jj = j + u * JSTEP;
                        if (jj >= NP) break;
                        if (!put(cv)) { ok = false; break; }
                        convert_strip(qb[u], s_lo, s_hi, GROUPED, cv);      // before the wait for the second slot
                        if (!put(cv)) { ok = false; break; }
                        if (JSTEP == 2) { s += 2; if (s >= (uint32_t) L::STAGES) { s -= L::STAGES; ph ^= 1; } }     // the other warps' pair
                        fetch(jj + 2 * JSTEP, qa[u], qb[u], qs[u]);
                        if (GROUPED) scale_pair(qs[u ^ 1], s_lo, s_hi);     // the next pair's first stage, converted before its slot is waited for
                        convert_strip(qa[u ^ 1], s_lo, s_hi, GROUPED, cv);
                    }
                }
            };
            if (a.grouped) run(std::true_type()); else run(std::false_type());
        }
    }
    else if (warp == NDQ)
    {
        if (lane == 0)
        {
            uint32_t tile_n = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < nitems && ok; item += gridDim.x, ++tile_n)
            {
                const int pos0 = a.rbt[4 * (item / NCT) + 1], n = a.rbt[4 * (item / NCT) + 2];
                // boxes of 64 rows: a row block with few picks brings in only the rows the MMA reads (n rounded up to 16 <= 64 nb)
                const int nb = (n + 63) >> 6;
                for (int kb = 0; kb < KBT; ++kb)
                {
                    const uint32_t it = tile_n * (uint32_t) KBT + kb, s = it % L::STAGES;
                    { PROBE_T0(); const bool w_ = it < (uint32_t) L::STAGES || mbar_wait(empty + s * 8, ((it / L::STAGES) - 1) & 1, abort_flag, a.status); PROBE_ADD(6); if (!w_) { ok = false; break; } }
                    mbar_expect_tx(full_b + s * 8, (uint32_t) nb * (TB * TK * 2));
                    for (int b = 0; b < nb; ++b)
                        tma_load_2d(sbase + s * L::STAGE + NMAT * L::A_BYTES + b * (TB * TK * 2), &tmap, kb * 64, pos0 + b * TB, full_b + s * 8);
                }
            }
        }
    }
    else if (warp == NDQ + 1)
    {
        if (lane == 0)
        {
            uint32_t tile_n = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < nitems && ok; item += gridDim.x, ++tile_n)
            {
                const int n = a.rbt[4 * (item / NCT) + 2];
                const uint32_t n16 = (uint32_t) ((n + 15) & ~15);
                const uint32_t idesc = (1u << 4) | ((n16 >> 3) << 17) | ((uint32_t) (TM >> 4) << 24);
                const uint32_t acc = tile_n % NACC, tacc = tmem + acc * 256;
                // the accumulator set is free once the tile that used it last has been read out
                { PROBE_T0(); const bool w_ = tile_n < (uint32_t) NACC || mbar_wait(tmem_free + acc * 8, ((tile_n / NACC) - 1) & 1, abort_flag, a.status); PROBE_ADD(2); if (!w_) break; }
                tc_fence_after();
                for (int kb = 0; kb < KBT && ok; ++kb)
                {
                    const uint32_t it = tile_n * (uint32_t) KBT + kb, s = it % L::STAGES, ph = (it / L::STAGES) & 1;
                    { PROBE_T0(); const bool w_ = mbar_wait(full_a + s * 8, ph, abort_flag, a.status); PROBE_ADD(0); if (!w_) { ok = false; break; } }
                    { PROBE_T0(); const bool w_ = mbar_wait(full_b + s * 8, ph, abort_flag, a.status); PROBE_ADD(1); if (!w_) { ok = false; break; } }
                    tc_fence_after();
                    const uint32_t at = sbase + s * L::STAGE, bt = at + NMAT * L::A_BYTES;
                    #pragma unroll
                    for (int k = 0; k < 4; ++k)
                    {
                        const uint64_t bd = smem_desc_sw128(bt + k * 32);
                        mma_f16_ss(tacc, smem_desc_sw128(at + k * 32), bd, idesc, (kb | k) != 0);
                        if (NMAT == 2) mma_f16_ss(tacc + 256, smem_desc_sw128(at + L::A_BYTES + k * 32), bd, idesc, (kb | k) != 0);
                    }
                    tc_commit(empty + s * 8);
                }
                if (ok) tc_commit(done + acc * 8);
            }
        }
    }
    else
    {
        // ---- read-out: warp NDQ + 2 + i reads the tensor-memory lanes of quarter (warp % 4) (a warp may only touch the quarter
        // that matches its number), i.e. 32 output channels, for all picks of the tile, 16 columns at a time. gate_up: SiLU(gate)
        // * up * routing weight -> fp16 activations; down: out[token] += scale * sum, one fp32 reduction per element (32 lanes =
        // 32 consecutive channels = 128 contiguous bytes). Because these warps do nothing else, the read-out of a tile overlaps
        // the dequantisation and (down: second accumulator set) the MMAs of the next one.
        const int lq = warp & 3, chalf = (warp - (NDQ + 2)) >> 2;        // lane quarter; gate_up: which half of the columns
        uint32_t tile_n = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < nitems && ok; item += gridDim.x, ++tile_n)
        {
            if (*abort_flag) break;
            const int rb = item / NCT, ct = item % NCT;
            const int e = a.rbt[4 * rb], pos0 = a.rbt[4 * rb + 1], n = a.rbt[4 * rb + 2];
            (void) chalf;
            const uint32_t acc = (uint32_t) (tile_n % NACC);
            const uint32_t n16 = (uint32_t) ((n + 15) & ~15);
            const int ch = ct * TM + lq * 32 + lane;
            const int chp = (ch & ~63) + operand_pos(ch & 63);       // where the down GEMM expects this channel of the activations
            const uint32_t tacc = tmem + acc * 256 + ((uint32_t) (lq * 32) << 16);
            const int csplit = NMAT == 2 ? (((int) n16 + 31) >> 5) << 4 : (int) n16;      // gate_up: columns [0, csplit) and [csplit, n16)
            const int cbeg = chalf ? csplit : 0, cend = chalf ? (int) n16 : csplit;
            // Everything the read-out needs besides the sums is fetched BEFORE the wait for the tile's last MMA, so that no global
            // load stands between that MMA and the release of the accumulators: the row scales, and in gate_up the
            // routing weights of the warp's columns (lane l holds picks cbeg + 32 i + l).
            float sc0 = 1.f, sc1 = 1.f;
            if (!a.grouped || (a.sh_i8 && e >= a.n_local))      // one fp32 scale per output row: applied here, not in the operand
            {
                const void* s0p = e < a.n_local ? (const void*) a.s0[e] : a.sh_s0;
                sc0 = __ldg((const float*) s0p + ch);
                if (NMAT == 2) { const void* s1p = e < a.n_local ? (const void*) a.s1[e] : a.sh_s1; sc1 = __ldg((const float*) s1p + ch); }
            }
            float wv[4] = {0.f, 0.f, 0.f, 0.f};
            if constexpr (NMAT == 2)
            {
                #pragma unroll
                for (int i = 0; i < 4; ++i) { const int pj = cbeg + 32 * i + lane; if (pj < n) wv[i] = __ldg(a.wt + pos0 + pj); }
            }
            { PROBE_T0(); const bool w_ = mbar_wait(done + acc * 8, (tile_n / NACC) & 1, abort_flag, a.status); if (PROBE_ON(threadIdx.x == (NDQ + 2) * 32)) PROBE_ADD(7); if (!w_) break; }
            PROBE_T0();
            tc_fence_after();
            if constexpr (NMAT == 2)
            {
                // Eight columns at a time, one register set: with 72 registers per thread a second set in flight (the next eight columns'
                // tensor-memory loads under the current eight's arithmetic) left the compiler too few registers to run the eight columns'
                // exp / reciprocal / product chains side by side, and the read-out took twice as long (measured: 127 M against 62 M
                // cycles per step over all SMs; the loads alone are 17 M). The tensor core waits for this read-out.
                // The loops carry no branch per column: a conditional region per column costs convergence-barrier instructions that
                // run one after the other (measured: ~70 cycles per column); the arithmetic runs for the padding columns too and
                // only the store is predicated; the int8 mode is a compile-time variant of the whole loop.
                uint32_t g0[8], u0[8];
                auto read_out = [&](auto aq_tag) {
                    constexpr bool AQ = decltype(aq_tag)::value;
                    auto emit = [&](const uint32_t (&gr)[8], const uint32_t (&ur)[8], int c0) {
                        const int rel = c0 - cbeg, wi = rel >> 5, lb = rel & 31;
                        const float wsel = wi == 0 ? wv[0] : wi == 1 ? wv[1] : wi == 2 ? wv[2] : wv[3];
                        float ws[8];
                        #pragma unroll
                        for (int j = 0; j < 8; ++j) ws[j] = __shfl_sync(0xffffffffu, wsel, lb + j);
                        #pragma unroll
                        for (int j = 0; j < 8; ++j)
                        {
                            const int p = c0 + j;
                            const float w = ws[j];
                            const float gg = __uint_as_float(gr[j]) * sc0, uu = __uint_as_float(ur[j]) * sc1;
                            if (AQ)
                            {
                                float v = gg / (1.f + expf(-gg)) * uu * w;
                                // second int8 round trip of the CPU engine: 32 consecutive channels = this warp
                                float m = fabsf(v);
                                #pragma unroll
                                for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
                                const float sq8 = m > 0.f ? __fdiv_rn(m, 127.f) : 1.f;
                                v = __fmul_rn((float) __float2int_rn(__fmul_rn(v, __fdiv_rn(1.f, sq8))), sq8);
                                // code x scale does not fit fp16: keep it as hi + lo halves, the down GEMM walks both
                                const __half hi = __float2half_rn(v), lo = __float2half_rn(v - __half2float(hi));
                                __half* dst = a.act + (size_t) (pos0 + p) * (2 * a.N) + chp;
                                if (p < n) { dst[0] = hi; dst[a.N] = lo; }
                            }
                            else
                            {
                                // fp16 result: the fast exponential and division are far inside its rounding (the reference's
                                // kernels make the same choice, runtime/tier/moe4/moe4t.cu:404-425 built with fast-math)
                                const __half v = __float2half_rn(__fdividef(gg, 1.f + __expf(-gg)) * uu * w);
                                if (p < n) a.act[(size_t) (pos0 + p) * a.N + chp] = v;
                            }
                        }
                    };
                    for (int c0 = cbeg; c0 < cend; c0 += 8)
                    {
                        tmem_ld8(tacc + c0, g0); tmem_ld8(tacc + 256 + c0, u0);
                        tmem_ld_wait();
                        emit(g0, u0, c0);
                    }
                };
                if (a.act_quant) read_out(std::true_type()); else read_out(std::false_type());
            }
            else
            {
                // Sixteen columns at a time, two register sets in turn: the tensor-memory load of the next sixteen columns is in
                // flight while the current sixteen go out as reductions. No branch per column here either: the padding columns
                // add 0 to the row of the block's last pick.
                uint32_t r0[16], r1[16];
                auto read_out = [&](auto peer_tag) {
                    constexpr bool PEER = decltype(peer_tag)::value;
                    auto emit = [&](const uint32_t (&r)[16], int c0, int tj) {
                        int tks[16];
                        #pragma unroll
                        for (int j = 0; j < 16; ++j) tks[j] = __shfl_sync(0xffffffffu, tj, j);
                        #pragma unroll
                        for (int j = 0; j < 16; ++j)
                        {
                            const int tk = tks[j];
                            const float v = c0 + j < n ? __uint_as_float(r[j]) * sc0 : 0.f;
                            if (PEER)
                            {
                                // the row's owner may be another GPU, and up to eight GPUs add into the same addresses: the
                                // reduction has to be atomic at system scope (a gpu-scope one is only atomic among this GPU's threads)
                                const int pr = tk / a.rows_per_rank;
                                red_add_sys(a.out_peer[pr] + (size_t) (tk - pr * a.rows_per_rank) * a.N + ch, v);
                            }
                            else atomicAdd(a.out + (size_t) tk * a.N + ch, v);
                        }
                    };
                    // lane j (and j + 16) fetches the token of pick c0 + j while the tensor-memory load is in flight
                    auto token_of = [&](int c0) { return __ldg(a.tok + pos0 + min(c0 + (lane & 15), n - 1)); };
                    if (cbeg < cend) tmem_ld16(tacc + cbeg, r0);
                    for (int c0 = cbeg; c0 < cend; c0 += 32)
                    {
                        const int ta = token_of(c0), tb = token_of(c0 + 16);
                        tmem_ld_wait();
                        if (c0 + 16 < cend) tmem_ld16(tacc + c0 + 16, r1);
                        emit(r0, c0, ta);
                        if (c0 + 16 < cend)
                        {
                            tmem_ld_wait();
                            if (c0 + 32 < cend) tmem_ld16(tacc + c0 + 32, r0);
                            emit(r1, c0 + 16, tb);
                        }
                    }
                };
                if (a.rows_per_rank) read_out(std::true_type()); else read_out(std::false_type());
            }
            tc_fence_before();
            __syncwarp();
            mbar_arrive_if(tmem_free + acc * 8, lane == 0);
            if (PROBE_ON(threadIdx.x == (NDQ + 2) * 32)) PROBE_ADD(8);
        }
    }
#ifdef HMOE_PROBE_WAITS
    if (threadIdx.x == 0) PROBE_ADD(15);
    #pragma unroll
    for (int i = 0; i < 16; ++i) if (pacc_[i]) atomicAdd(&g_probe[(NMAT - 1) * 32 + i], pacc_[i]);
#endif
    tc_fence_before();
    __syncthreads();
    if (warp == NDQ + 1)
    {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

typedef CUresult (*encode_fn_t)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

encode_fn_t encode_fn()
{
    static encode_fn_t f = nullptr;
    if (!f)
    {
        void* p = nullptr; cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess) f = (encode_fn_t) p;
    }
    return f;
}

// row-major fp16 [rows][K] in boxes of 64 columns x 64 rows, 128-byte swizzle
bool make_map(CUtensorMap* m, const void* ptr, int K, size_t rows)
{
    encode_fn_t f = encode_fn();
    if (!f) return false;
    cuuint64_t dims[2] = {(cuuint64_t) K, (cuuint64_t) rows};
    cuuint64_t strides[1] = {(cuuint64_t) K * 2};
    cuuint32_t box[2] = {TK, TB}, es[2] = {1, 1};
    return f(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*) ptr, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

size_t up256(size_t b) { return (b + 255) / 256 * 256; }

// the kernels' dynamic shared memory exceeds the default limit: raise it once per device
void set_gemm_attributes()
{
    static DeviceOnce once;
    if (!once.first()) return;
    cudaFuncSetAttribute(prefill_gemm_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, PfSmem<2>::total);
    cudaFuncSetAttribute(prefill_gemm_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, PfSmem<1>::total);
}

struct WsLayout
{
    size_t status, plan, counts, offs, hist, order, tok, eid, wt, rbt, xg, act, total;
    int nblocks, rows_cap, maxrb;
};

WsLayout ws_layout(int R, int topk, int n_local, int H, int I, int bm, int kfold = 1)
{
    WsLayout w;
    const size_t P = (size_t) R * topk;
    w.nblocks = (int) ((P + CHUNK - 1) / CHUNK);
    w.rows_cap = (int) (P + R);
    w.maxrb = (int) ((P + R) / bm + n_local + 2);
    size_t o = 0;
    w.status = o; o += 256;
    w.plan = o; o += 256;
    w.counts = o; o += up256((size_t) (n_local + 2) * 4);
    w.offs = o; o += up256((size_t) (n_local + 3) * 4);
    w.hist = o; o += up256((size_t) w.nblocks * (n_local > 0 ? n_local : 1) * 4);
    w.order = o; o += up256((size_t) w.rows_cap * 4);
    w.tok = o; o += up256((size_t) w.rows_cap * 4);
    w.eid = o; o += up256((size_t) w.rows_cap * 4);
    w.wt = o; o += up256((size_t) w.rows_cap * 4);
    w.rbt = o; o += up256((size_t) w.maxrb * 16);
    w.xg = o; o += up256((size_t) w.rows_cap * H * 2 * kfold);
    w.act = o; o += up256((size_t) w.rows_cap * I * 2 * kfold);
    w.total = o;
    return w;
}

int run_permute(const int64_t* sel, const void* rw, int R, int topk, int lo, int n_local, int shared_rows, int shared_row0, int bm, int balance,
                int* counts, int* offs, int* hist, int nblocks, int* order, int* tok, int* eid, float* wt, int* rbt, Plan* plan, cudaStream_t st)
{
    const int P = R * topk;
    permute_hist_kernel<<<nblocks, 32, 0, st>>>(sel, P, lo, n_local, hist);
    permute_scan_kernel<<<1, 256, 0, st>>>(hist, nblocks, n_local, shared_rows, bm, balance, counts, offs, rbt, plan);
    const int sb = shared_rows > 0 ? (shared_rows + CHUNK - 1) / CHUNK : 0;
    permute_scatter_kernel<<<nblocks + sb, 32, 0, st>>>(sel, (const __half*) rw, P, topk, lo, n_local, shared_rows, shared_row0, hist, offs, nblocks, order, tok, eid, wt);
    count_launches(3);
    return cudaGetLastError() == cudaSuccess ? HMOE_OK : fail(HMOE_E_CUDA, "hmoe_permute: launch failed");
}

}  // namespace

size_t prefill_ws_bytes(int R, int topk, int n_local, int H, int I, int act_quant) { return ws_layout(R, topk, n_local, H, I, TN, act_quant ? 2 : 1).total; }

namespace {
__global__ void set_plan_kernel(Plan* plan, int total, int nrb) { plan->total = total; plan->nrb = nrb; plan->pad[0] = plan->pad[1] = 0; }
}

// The reference's calling convention (moe4t.forward, runtime/tier/moe4/moe4t.cu:498-524): the caller has already sorted the
// picks by expert (tok, wt in that order) and built the row-block table; npos picks, nrb row blocks of <= 256 picks.
size_t prefill_sorted_ws_bytes(int npos, int H, int I, int act_quant)
{
    const int f = act_quant ? 2 : 1;
    return 512 + up256((size_t) npos * H * 2 * f) + up256((size_t) npos * I * 2 * f);
}

int prefill_sorted_launch(const hmoe_layer* L, const void* x, int x_dtype, const int32_t* tok, const float* wt, const int32_t* rbt, int nrb,
                          int npos, int n_local, int act_quant, float* out, void* ws, size_t ws_bytes, cudaStream_t st)
{
    const int H = L->H, I = L->I;
    if (npos < 0 || nrb < 0) return fail(HMOE_E_ARG, "hmoe_prefill_sorted: sizes");
    if (npos == 0 || nrb == 0) return HMOE_OK;
    if (H % 128 || I % 128 || H < 128 || I < 128) return fail(HMOE_E_ARG, "hmoe_prefill_sorted: H and I must be multiples of 128");
    if (!(L->group == 0 && L->scale_dtype == HMOE_F32) && !(L->group == 128 && L->scale_dtype == HMOE_BF16))
        return fail(HMOE_E_ARG, "hmoe_prefill_sorted: scales must be fp32 per row (group 0) or bf16 per 128 columns");
    if (x_dtype != HMOE_F16 && x_dtype != HMOE_BF16) return fail(HMOE_E_ARG, "hmoe_prefill_sorted: x must be fp16 or bf16");
    if (!x || !tok || !wt || !rbt || !out || !ws) return fail(HMOE_E_ARG, "hmoe_prefill_sorted: null pointer");
    const int kf = act_quant ? 2 : 1;
    if (ws_bytes < prefill_sorted_ws_bytes(npos, H, I, act_quant)) return fail(HMOE_E_WS, "hmoe_prefill_sorted: workspace too small");
    const int sms = device_sms();
    if (sms <= 0) return fail(HMOE_E_CUDA, "hmoe_prefill_sorted: no current CUDA device");
    set_gemm_attributes();
    char* b = (char*) ws;
    unsigned* status = (unsigned*) b;
    Plan* plan = (Plan*) (b + 256);
    __half* xg = (__half*) (b + 512);
    __half* act = (__half*) (b + 512 + up256((size_t) npos * H * 2 * kf));
    set_plan_kernel<<<1, 1, 0, st>>>(plan, npos, nrb);
    gather_kernel<<<npos, 192, 0, st>>>(x, x_dtype == HMOE_BF16, tok, plan, H, act_quant, xg);
    CUtensorMap mx, ma;
    if (!make_map(&mx, xg, H * kf, (size_t) npos) || !make_map(&ma, act, I * kf, (size_t) npos)) return fail(HMOE_E_CUDA, "hmoe_prefill_sorted: cuTensorMapEncodeTiled failed");
    GemmArgs g;
    g.grouped = L->group != 0; g.act_quant = act_quant; g.n_local = n_local; g.kfold = kf;
    g.sh_i8 = L->shared_format == 1 && L->sh_gate_w != nullptr;
    g.plan = plan; g.rbt = rbt; g.tok = tok; g.wt = wt; g.act = act; g.out = out; g.status = status;
    g.rows_per_rank = 0;
    for (int p = 0; p < 8; ++p) g.out_peer[p] = nullptr;
    g.K = H; g.N = I; g.w0 = L->gate_w; g.w1 = L->up_w; g.s0 = L->gate_s; g.s1 = L->up_s;
    g.sh_w0 = L->sh_gate_w; g.sh_w1 = L->sh_up_w; g.sh_s0 = L->sh_gate_s; g.sh_s1 = L->sh_up_s;
    prefill_gemm_kernel<2><<<sms, pf_threads(2), PfSmem<2>::total, st>>>(mx, g);
    g.K = I; g.N = H; g.w0 = L->down_w; g.w1 = nullptr; g.s0 = L->down_s; g.s1 = nullptr;
    g.sh_w0 = L->sh_down_w; g.sh_w1 = nullptr; g.sh_s0 = L->sh_down_s; g.sh_s1 = nullptr;
    prefill_gemm_kernel<1><<<sms, pf_threads(1), PfSmem<1>::total, st>>>(ma, g);
    count_launches(4);
    const cudaError_t err = cudaGetLastError();
    return err == cudaSuccess ? HMOE_OK : fail(HMOE_E_CUDA, cudaGetErrorString(err));
}

int permute_launch(const int64_t* sel, const void* rw, int R, int topk, int lo, int n_local, int shared_rows, int bm, int balance,
                   int32_t* order, int32_t* tok, int32_t* eid, float* wt, int32_t* counts, int32_t* rbt, int32_t* plan2, void* ws, size_t ws_bytes,
                   cudaStream_t st)
{
    if (R < 1 || topk < 1 || n_local < 1 || n_local > 256 || bm < 1) return fail(HMOE_E_ARG, "hmoe_permute: needs R >= 1, 1 <= n_local <= 256, bm >= 1");
    if (!sel || !rw || !tok || !eid || !wt || !counts || !rbt || !plan2 || !ws) return fail(HMOE_E_ARG, "hmoe_permute: null pointer");
    const size_t P = (size_t) R * topk;
    const int nblocks = (int) ((P + CHUNK - 1) / CHUNK);
    const size_t need = up256((size_t) nblocks * n_local * 4) + up256((size_t) (n_local + 3) * 4);
    if (ws_bytes < need) return fail(HMOE_E_WS, "hmoe_permute: workspace too small");
    int* hist = (int*) ws;
    int* offs = (int*) ((char*) ws + up256((size_t) nblocks * n_local * 4));
    return run_permute(sel, rw, R, topk, lo, n_local, shared_rows, 0, bm, balance, counts, offs, hist, nblocks, order, tok, eid, wt, rbt, (Plan*) plan2, st);
}

size_t permute_ws_bytes(int R, int topk, int n_local)
{
    const size_t P = (size_t) R * topk;
    const int nblocks = (int) ((P + CHUNK - 1) / CHUNK);
    return up256((size_t) nblocks * n_local * 4) + up256((size_t) (n_local + 3) * 4);
}

int prefill_launch(const hmoe_layer* L, const void* x, int x_dtype, const int64_t* sel, const void* rw, int R, int lo, int n_local,
                   int act_quant, float* out, void* ws, size_t ws_bytes, cudaStream_t st, int shared_row0, int shared_rows,
                   void* const* out_peer, int world, int rows_per_rank)
{
    if (shared_rows < 0) { shared_row0 = 0; shared_rows = R; }
    if (out_peer && (world < 1 || world > 8 || rows_per_rank < 1 || (long long) world * rows_per_rank < R))
        return fail(HMOE_E_ARG, "hmoe_prefill_ep_peer: world must be 1..8 and world * rows_per_rank must cover the rows");          // default: the shared expert takes every row
    if (shared_row0 < 0 || shared_row0 + shared_rows > R) return fail(HMOE_E_ARG, "hmoe_prefill: shared row range outside the rows");
    const int H = L->H, I = L->I;
    if (R < 1) return fail(HMOE_E_ARG, "hmoe_prefill: rows must be >= 1");
    if (L->topk < 1 || L->topk > TOPK_MAX) return fail(HMOE_E_ARG, "hmoe_prefill: topk must be 1..8");
    if (H % 128 || I % 128 || H < 128 || I < 128) return fail(HMOE_E_ARG, "hmoe_prefill: H and I must be multiples of 128");
    if (n_local < 1 || n_local > 256) return fail(HMOE_E_ARG, "hmoe_prefill: 1..256 local experts");
    if (!(L->group == 0 && L->scale_dtype == HMOE_F32) && !(L->group == 128 && L->scale_dtype == HMOE_BF16))
        return fail(HMOE_E_ARG, "hmoe_prefill: scales must be fp32 per row (group 0) or bf16 per 128 columns");
    if (x_dtype != HMOE_F16 && x_dtype != HMOE_BF16) return fail(HMOE_E_ARG, "hmoe_prefill: x must be fp16 or bf16");
    if (!x || !sel || !rw || (!out && !out_peer) || !ws) return fail(HMOE_E_ARG, "hmoe_prefill: null pointer");
    const int kf = act_quant ? 2 : 1;
    const WsLayout w = ws_layout(R, L->topk, n_local, H, I, TN, kf);
    if (ws_bytes < w.total) return fail(HMOE_E_WS, "hmoe_prefill: workspace too small (the int8 mode needs hmoe_prefill_ws_bytes(..., act_quant = 1))");
    const int sms = device_sms();
    if (sms <= 0) return fail(HMOE_E_CUDA, "hmoe_prefill: no current CUDA device");
    set_gemm_attributes();
    char* b = (char*) ws;
    unsigned* status = (unsigned*) (b + w.status);
    Plan* plan = (Plan*) (b + w.plan);
    int* counts = (int*) (b + w.counts); int* offs = (int*) (b + w.offs); int* hist = (int*) (b + w.hist);
    int* order = (int*) (b + w.order); int* tok = (int*) (b + w.tok); int* eid = (int*) (b + w.eid); float* wt = (float*) (b + w.wt);
    int* rbt = (int*) (b + w.rbt);
    __half* xg = (__half*) (b + w.xg); __half* act = (__half*) (b + w.act);
    const int has_shared = L->sh_gate_w != nullptr;
    int rc = run_permute(sel, rw, R, L->topk, lo, n_local, has_shared ? shared_rows : 0, shared_row0, TN, 1, counts, offs, hist, w.nblocks, order, tok, eid, wt,
                         rbt, plan, st);
    if (rc) return rc;
    gather_kernel<<<w.rows_cap, 192, 0, st>>>(x, x_dtype == HMOE_BF16, tok, plan, H, act_quant, xg);
    CUtensorMap mx, ma;
    if (!make_map(&mx, xg, H * kf, (size_t) w.rows_cap) || !make_map(&ma, act, I * kf, (size_t) w.rows_cap)) return fail(HMOE_E_CUDA, "hmoe_prefill: cuTensorMapEncodeTiled failed");
    GemmArgs g;
    g.grouped = L->group != 0; g.act_quant = act_quant; g.n_local = n_local; g.kfold = kf;
    g.sh_i8 = L->shared_format == 1 && L->sh_gate_w != nullptr;
    g.plan = plan; g.rbt = rbt; g.tok = tok; g.wt = wt; g.act = act; g.out = out; g.status = status;
    g.rows_per_rank = out_peer ? rows_per_rank : 0;
    for (int p = 0; p < 8; ++p) g.out_peer[p] = (out_peer && p < world) ? (float*) out_peer[p] : nullptr;
    g.K = H; g.N = I; g.w0 = L->gate_w; g.w1 = L->up_w; g.s0 = L->gate_s; g.s1 = L->up_s;
    g.sh_w0 = L->sh_gate_w; g.sh_w1 = L->sh_up_w; g.sh_s0 = L->sh_gate_s; g.sh_s1 = L->sh_up_s;
    prefill_gemm_kernel<2><<<sms, pf_threads(2), PfSmem<2>::total, st>>>(mx, g);
    g.K = I; g.N = H; g.w0 = L->down_w; g.w1 = nullptr; g.s0 = L->down_s; g.s1 = nullptr;
    g.sh_w0 = L->sh_down_w; g.sh_w1 = nullptr; g.sh_s0 = L->sh_down_s; g.sh_s1 = nullptr;
    prefill_gemm_kernel<1><<<sms, pf_threads(1), PfSmem<1>::total, st>>>(ma, g);
    count_launches(3);
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return fail(HMOE_E_CUDA, cudaGetErrorString(err));
    return HMOE_OK;
}

}  // namespace hmoe

#ifdef HMOE_PROBE_WAITS
extern "C" int hmoe_probe_read(unsigned long long* out, int clear)
{
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out, hmoe::g_probe, sizeof(unsigned long long) * 64);
    if (clear) { unsigned long long z[64] = {}; cudaMemcpyToSymbol(hmoe::g_probe, z, sizeof(z)); }
    return 0;
}
#endif

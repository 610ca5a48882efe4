// Shared device helpers of the MoE expert kernels (sm_100a): bounded mbarrier waits, 1-D bulk copies into shared memory,
// the int4 -> fp16 fragment conversion and the m16n8k16 MMA wrapper.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace hmoe {

// status word bits written by kernels (device) and read by the host on request
enum : unsigned { ST_WAIT_TIMEOUT = 1u, ST_BAD_INDEX = 2u };

constexpr int TOPK_MAX = 8;
constexpr int MAXR = 16;                  // decode rows per call (tokens x (1 + MTP drafts))
constexpr int MAXS = MAXR * TOPK_MAX + 1; // distinct experts of a decode call + the shared expert
constexpr int MAXT = MAXR * TOPK_MAX + 2; // 8-row tiles: at most one per pick, two for a 16-row shared expert
constexpr int MAXB = 256;                 // blocks of a streaming kernel (one per SM)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t) __cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, int count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// arrive by the threads whose `on` is set, as a predicated instruction (no branch around it)
__device__ __forceinline__ void mbar_arrive_if(uint32_t bar, bool on)
{
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %1, 0;\n @p mbarrier.arrive.shared::cta.b64 _, [%0];\n}\n" ::"r"(bar), "r"((uint32_t) on) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// try_wait that lets the hardware park the thread for up to `hint_ns` before it reports failure (fewer polls issued)
__device__ __forceinline__ bool mbar_try_hint(uint32_t bar, uint32_t parity, uint32_t hint_ns)
{
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity), "r"(hint_ns) : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long globaltimer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait: gives up after about `limit_ns` of wall time, raises the abort flag in shared memory and the timeout bit
// of the global status word, and returns false. Every waiter checks the abort flag, so after one timeout the whole
// block drains quickly instead of spinning.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, unsigned* status,
                                          unsigned long long limit_ns = 1000000000ull)
{
    if (mbar_try(bar, parity)) return true;
    unsigned long long t0 = 0;
    for (uint32_t i = 0;; ++i)
    {
        if (mbar_try_hint(bar, parity, 20000u)) return true;
        if ((i & 63u) == 63u)
        {
            if (*abort_flag) return false;
            const unsigned long long now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit_ns) break;
        }
    }
    *abort_flag = 1;
    if (status) atomicOr(status, ST_WAIT_TIMEOUT);
    return false;
}
// Diagnostic build (-DHMOE_PROBE_TIMELINE): kernels of the decode chain stamp the global timer at a few points (earliest and latest
// over the blocks); every source file has its own table and reader. Not part of the normal build.
#ifdef HMOE_PROBE_TIMELINE
static __device__ unsigned long long g_tl[16];
#define TL_MIN(i) do { if (threadIdx.x == 0) atomicMin(&g_tl[i], globaltimer_ns()); } while (0)
#define TL_MAX(i) do { if (threadIdx.x == 0) atomicMax(&g_tl[i], globaltimer_ns()); } while (0)
#define TL_READER(name) extern "C" int name(unsigned long long* out, int clear) { \
    cudaDeviceSynchronize(); cudaMemcpyFromSymbol(out, g_tl, sizeof(unsigned long long) * 16); \
    if (clear) { unsigned long long z[16]; for (int i = 0; i < 16; ++i) z[i] = (i & 1) ? 0ull : ~0ull; cudaMemcpyToSymbol(g_tl, z, sizeof(z)); } return 0; }
#else
#define TL_MIN(i)
#define TL_MAX(i)
#define TL_READER(name)
#endif
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// 1-D bulk copy global -> shared (both 16-byte aligned, size a multiple of 16), completion counted on an mbarrier.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__device__ __forceinline__ uint4 lds128(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 ldg128_nc(const void* p)
{
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
// plain (coherent) 16-byte load, for data written by an earlier kernel of the same call
__device__ __forceinline__ uint4 ldg128(const void* p)
{
    uint4 v;
    asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_f16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1)
{
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// One 32-bit word of packed codes = the A fragment of one 16-column step for this lane: nibble i holds
// (column pair member i >> 2, column half (i >> 1) & 1, row half i & 1). Returns the four fp16x2 registers
// {(row g, k 2q..2q+1), (row g+8, same k), (row g, k 2q+8..), (row g+8, k 2q+8..)} with value code - 8, exactly.
// (1024 + c is exact in fp16; the nibbles that sit four bits higher give 1024 + 16 c and are brought back by one fused
// multiply-add with 1/16 and -72.)
// This is the magic-number conversion the reference's decode kernels use for the same words (dec8, runtime/tier/moe4/moe4.cu:56-67):
// the stored nibble order was chosen for exactly these two masks, so any converter for this layout extracts the same pairs;
// a byte-permute (prmt) variant needs one more instruction per word and was not kept.
__device__ __forceinline__ void frag_from_codes(uint32_t w, uint32_t* a)
{
    // Written as PTX with plain 32-bit immediates: half2 constants built through the cuda_fp16 helpers are re-materialised
    // at every use (measured: six extra integer instructions per word).
    const uint32_t w8 = w >> 8;
    uint32_t lo0, hi0, lo1, hi1;
    asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(lo0) : "r"(w));     // (w & mask) | 1024.0 in both halves
    asm("lop3.b32 %0, %1, 0x00f000f0, 0x64006400, 0xea;" : "=r"(hi0) : "r"(w));
    asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(lo1) : "r"(w8));
    asm("lop3.b32 %0, %1, 0x00f000f0, 0x64006400, 0xea;" : "=r"(hi1) : "r"(w8));
    asm("sub.f16x2 %0, %1, %2;" : "=r"(a[0]) : "r"(lo0), "r"(0x64086408u));                            // - 1032
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(a[1]) : "r"(hi0), "r"(0x2c002c00u), "r"(0xd480d480u));   // / 16 - 72
    asm("sub.f16x2 %0, %1, %2;" : "=r"(a[2]) : "r"(lo1), "r"(0x64086408u));
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(a[3]) : "r"(hi1), "r"(0x2c002c00u), "r"(0xd480d480u));
}

// The reference's int8 format (its shared expert and dense linears, runtime/core/hecate_runtime.py:38-48): value = code - 128.
// 4 bytes (c0 rh0, c0 rh1, c1 rh0, c1 rh1) -> fp16x2 (row g: c0, c1) and (row g + 8: c0, c1), value code - 128, exactly
// (the same magic-number step as the reference uses for these bytes, runtime/tier/moe4/moe4.cu:48-55: 1024 + code is exact in fp16)
__device__ __forceinline__ void dec_i8(uint32_t w, uint32_t& lo, uint32_t& hi)
{
    uint32_t h0, h1;
    asm("lop3.b32 %0, %1, 0x00ff00ff, 0x64006400, 0xea;" : "=r"(h0) : "r"(w));
    asm("lop3.b32 %0, %1, 0x00ff00ff, 0x64006400, 0xea;" : "=r"(h1) : "r"(w >> 8));
    asm("sub.f16x2 %0, %1, %2;" : "=r"(lo) : "r"(h0), "r"(0x64806480u));
    asm("sub.f16x2 %0, %1, %2;" : "=r"(hi) : "r"(h1), "r"(0x64806480u));
}

// position of two-value word p (columns 2p, 2p+1 of a 64-column block) in the activation row order the kernels read:
// t = p / 8 (16-column step), h = (p % 8) / 4, q = p % 4  ->  q * 8 + t * 2 + h (the B-fragment order the reference's norm +
// router kernel may pre-write for moe4, frag_word, runtime/tier/moe4/moe4.cu:72)
__device__ __forceinline__ int frag_pos(int p) { return (p & 3) * 8 + (p >> 3) * 2 + ((p >> 2) & 1); }

__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) { return __uint_as_float((uint32_t) b << 16); }

// deterministic exp: the same sequence of correctly rounded operations as the CPU checker's routine, so selections that
// depend on it are reproducible bit for bit
__device__ __forceinline__ float det_expf(float x)
{
    x = fminf(fmaxf(x, -87.f), 88.f);
    const float t = __fmul_rn(x, 1.44269504088896341f);
    const float n = rintf(t);
    float r = __fmaf_rn(n, -0.693145751953125f, x);
    r = __fmaf_rn(n, -1.42860682030941723212e-6f, r);
    float p = 1.9875691500e-4f;
    p = __fmaf_rn(p, r, 1.3981999507e-3f);
    p = __fmaf_rn(p, r, 8.3334519073e-3f);
    p = __fmaf_rn(p, r, 4.1665795894e-2f);
    p = __fmaf_rn(p, r, 1.6666665459e-1f);
    p = __fmaf_rn(p, r, 5.0000001201e-1f);
    p = __fmaf_rn(p, __fmul_rn(r, r), r);
    p = __fadd_rn(p, 1.f);
    return __fmul_rn(p, __int_as_float(((int) n + 127) << 23));
}

// ---- expert-parallel exchange over peer memory: flag stores / loads at system scope, and the staging area every rank keeps
// for the decode dispatch (the step's rows, selections and weights at their global row positions, one flag per sending rank,
// two control words)
__device__ __forceinline__ void sys_st_release(unsigned* p, unsigned v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ unsigned sys_ld_acquire(const unsigned* p)
{
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
struct StageLayout
{
    size_t x, sel, rw, flags, ctl, total;
    __host__ __device__ StageLayout(int H, int topk)
    {
        x = 0; sel = x + (size_t) MAXR * H * 2; rw = sel + (size_t) MAXR * topk * 8; flags = (rw + (size_t) MAXR * topk * 2 + 255) / 256 * 256;
        ctl = flags + 256; total = ctl + 256;
    }
};

// ---- pieces of the residual + RMS-norm kernels (hmoe_combine_norm, hmoe_norm_router): 4-wide column arithmetic in the order
// the bit-identity contract with the reference norm kernels fixes (see sum_norm_kernel)
__device__ __forceinline__ float4 vec_add(float4 a, const float4 b) { a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w; return a; }
__device__ __forceinline__ float sq_accumulate(float s, const float4 v) { s = fmaf(v.x, v.x, s); s = fmaf(v.y, v.y, s); s = fmaf(v.z, v.z, s); return fmaf(v.w, v.w, s); }
__device__ __forceinline__ float butterfly32(float v)
{
    #pragma unroll
    for (int d = 16; d; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}
template <bool WBF>
__device__ __forceinline__ float4 norm_weight4(const uint16_t* w, int vec)
{
    const uint2 bits = *(const uint2*) (w + 4 * vec);
    if (WBF) return make_float4(__uint_as_float(bits.x << 16), __uint_as_float(bits.x & 0xffff0000u), __uint_as_float(bits.y << 16), __uint_as_float(bits.y & 0xffff0000u));
    const float2 lo = __half22float2(*(const __half2*) &bits.x), hi = __half22float2(*(const __half2*) &bits.y);
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}
// fp16x4 of (v * (w + cbias)) * k, each product rounded on its own as in the reference kernel
__device__ __forceinline__ uint2 norm_pack4(const float4 v, float4 w, float cbias, float k)
{
    if (cbias != 0.f) { w.x += cbias; w.y += cbias; w.z += cbias; w.w += cbias; }
    const __half2 lo = __floats2half2_rn(__fmul_rn(__fmul_rn(v.x, w.x), k), __fmul_rn(__fmul_rn(v.y, w.y), k));
    const __half2 hi = __floats2half2_rn(__fmul_rn(__fmul_rn(v.z, w.z), k), __fmul_rn(__fmul_rn(v.w, w.w), k));
    return make_uint2(*(const uint32_t*) &lo, *(const uint32_t*) &hi);
}

// Routing of one decode call, built once per call by the prepare kernel and read by the expert kernels.
// The distinct selected experts are taken in ascending id order (as the reference's in-kernel route() orders them,
// runtime/tier/moe4/moe4.cu:86-110), followed by the shared expert if there is one. Each expert's rows are cut into
// tiles of <= 8 rows: a tile is the unit the expert kernels work on (its rows are the 8 columns of the MMAs). An expert
// picked by more than 8 rows therefore appears as two tiles and is streamed twice (the second pass hits L2).
template <int NT, typename RowT = unsigned char>
struct RouteT
{
    int m;                          // distinct routed experts
    int ntiles;
    int pad[2];
    short expert[NT];               // local expert id of the tile (-1 = shared)
    unsigned char nrows[NT];        // rows in the tile (1..8)
    RowT rows[NT][8];               // their row numbers, ascending; entries >= nrows repeat the first row
    float w[NT][8];                 // routing weight per listed row (summed over repeated picks), 0 beyond nrows
    short rowbase[NT];              // number of real rows in the tiles before this one (row index of the tile's first row in
                                    // the per-pick buffers; at most rows * (topk + 1) real rows per call)
    int split[2][MAXB + 1];         // streaming kernels (0 gate_up, 1 down): block b works on items [split[b], split[b + 1])
};
using Route = RouteT<MAXT>;

// Short prefill: more rows than a decode call takes, still so few that most experts see fewer than eight of them, so the
// streaming kernels (every distinct expert read once at memory speed) beat the grouped tensor-core GEMMs (whose weight
// conversion costs the same for a 3-pick row block as for a 256-pick one). The reference has the same range between its
// decode and its grouped-GEMM paths (runtime/tier/tier_split.py:341-355: 9..64 rows through the moe4 decode kernels in 8-row
// chunks, each chunk streaming its experts again); here the whole call is one tile list, so an expert is streamed once per
// eight of its picks. A pick is one tile column (an expert picked twice by a row gets two columns of that row).
constexpr int SHORT_MAXR = 640;               // where the grouped GEMMs catch up on a 256-expert layer under uniform routing (row numbers and the rows
                                              // of the per-pick buffer are 16-bit in the route)
// tiles: one partial tile per local expert and for the shared expert, plus the full ones
constexpr int SHORT_MAXT = 256 + 1 + (SHORT_MAXR * TOPK_MAX) / 8 + SHORT_MAXR / 8 + 2;
using RouteShort = RouteT<SHORT_MAXT, unsigned short>;
constexpr int FORWARD_SHORT_ROWS = 384;     // hmoe_forward: calls of up to this many rows take the short path (uniform routing over 256
                                            // experts: level with the grouped GEMMs at 640 rows, 1.4 x faster at 384; skewed routing moves the crossing down)

constexpr int FORWARD_SHORT_ROWS_SH8 = 256; // the same with the reference's int8 shared expert (measured: 1.69 ms against 2.2 - 2.7 ms at 256 rows, level near 384)

}  // namespace hmoe

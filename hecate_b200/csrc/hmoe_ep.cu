// Expert-parallel exchange over NVLink peer memory for the decode path.
//
// The reference has no expert parallelism; its closest relative is the band mailbox: every band gets all rows plus
// (sel, rw), ignores foreign expert ids (runtime/tier/moe4/moe4.cu:93) and hands back an fp32 partial that the combine adds
// in a fixed order (runtime/tier/moe4/moe4.cu:702-717; slot + ISSUE / DONE flags in runtime/tier/rtx_graph.py:105-134).
// Here the bands are the GPUs of one box: rank r owns experts [r E / W, (r + 1) E / W), every rank sees the step's <= 16 rows
// (decode "dispatch" = the rows are replicated, each rank filters by expert id), computes its partial with the decode kernels
// into its slot of a symmetric buffer, and the combine is one kernel per rank that
// The step number (generation) lives in device memory: the step's prepare kernel bumps it, the down kernel picks the slot
// gen % 2 and the combine reads it, so a step has no host-side state and can be captured in a CUDA graph.
//   1. raises this rank's generation flag in every peer's memory (st.release.sys over NVLink),
//   2. waits, bounded, until every peer's flag in local memory has reached the generation,
//   3. reads every rank's partial (peer loads) and adds them to the layer output in rank order, the same order on every
//      rank, so all ranks hold bit-identical results,
//   4. clears the slot of the other parity for the step after next.
// Two slots alternate by step parity: a peer signals generation g + 1 only after its reads of generation g are done, so
// passing the wait for g + 1 proves nobody still reads the slot that step g + 2 will reuse.
#include <cstring>
#include "hmoe_common.cuh"
#include "hmoe_internal.h"

namespace hmoe {
namespace {

struct EpArgs
{
    int rank, world;
    float* slots[8];          // slots[p] = base of rank p's two partial slots (peer pointers; own pointer for p == rank)
    unsigned* flags[8];       // flags[p] = base of rank p's flag array [world]
};

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p)
{
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float4 ld_peer(const float4* p)
{
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}

// own_rows = 0: f [rows][H] += the sum over all rows (every rank ends with the whole batch, bit-identical). own_rows = 1 (tokens
// are data-parallel: rank r owns rows r, r + world, ...): f [own rows][H] += the sums of this rank's rows only, an eighth of the
// peer traffic at 8 GPUs; this is the combine half of the all-to-all.
__global__ void __launch_bounds__(256) ep_combine_kernel(const EpArgs a, const unsigned* __restrict__ gen_ptr, float* __restrict__ f, int n,
                                                         size_t slot_floats, unsigned* __restrict__ status, int own_rows, int H)
{
    __shared__ int ok_sh;
    // launched with programmatic stream serialization behind the down kernel (which releases its dependents early): the blocks are
    // resident when down ends; nothing is read, and above all no flag raised, before down has completed with its sums visible
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const unsigned gen = *gen_ptr;            // bumped by this step's prepare kernel, stable for the rest of the step
    const int parity = gen & 1;
    if (blockIdx.x == 0 && threadIdx.x < a.world) st_release_sys(a.flags[threadIdx.x] + a.rank, gen);
    if (threadIdx.x == 0)
    {
        int ok = 1;
        const unsigned long long t0 = globaltimer_ns();
        for (int p = 0; p < a.world && ok; ++p)
            while ((int) (ld_acquire_sys(a.flags[a.rank] + p) - gen) < 0)
                if (globaltimer_ns() - t0 > 2000000000ull) { ok = 0; atomicOr(status, ST_WAIT_TIMEOUT); break; }
        ok_sh = ok;
    }
    __syncthreads();
    if (!ok_sh) return;
    for (int i = (blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += gridDim.x * blockDim.x * 4)
    {
        *(float4*) (a.slots[a.rank] + (size_t) (parity ^ 1) * slot_floats + i) = make_float4(0.f, 0.f, 0.f, 0.f);
        int o = i;                                         // position in f
        if (own_rows)
        {
            const int r = i / H;
            if (r % a.world != a.rank) continue;
            o = (r / a.world) * H + (i - r * H);
        }
        // all peers' loads are issued before the first sum (a warp issues in order: a sum between two loads would serialise
        // the NVLink round trips); the sums then run in rank order
        float4 v[8];
        #pragma unroll
        for (int p = 0; p < 8; ++p)
            if (p < a.world) v[p] = ld_peer((const float4*) (a.slots[p] + (size_t) parity * slot_floats + i));
        float4 acc = *(float4*) (f + o);
        #pragma unroll
        for (int p = 0; p < 8; ++p)
            if (p < a.world) { acc.x += v[p].x; acc.y += v[p].y; acc.z += v[p].z; acc.w += v[p].w; }
        *(float4*) (f + o) = acc;
    }
}

// Decode dispatch: the all-gather half of the all-to-all, over peer memory. Tokens are data-parallel: rank r holds rows
// r, r + world, ... of the step's R rows (with the selections and weights its own router produced for them). Block p of the
// kernel stores this rank's rows into rank p's staging area at their global row positions (x as 16-byte words, then sel and
// rw), raises this rank's flag there with release semantics at system scope, and waits (bounded) until rank p has raised its
// flag here: when the kernel ends, the local staging area holds all R rows. The step number lives in the staging area's control
// words (the last block to finish advances it), so a step has no host state. One staging area suffices: a rank reaches its
// next dispatch only through its combine, which waits for every peer's combine flag, which a peer raises after the kernels
// that read its staging area.
struct StageArgs
{
    int rank, world;
    char* stage[8];
};
constexpr int DISPATCH_THREADS = 1024;

__global__ void __launch_bounds__(DISPATCH_THREADS) ep_dispatch_kernel(const StageArgs a, const uint4* __restrict__ x_own, const int64_t* __restrict__ sel_own,
                                                          const uint16_t* __restrict__ rw_own, int R, int H, int topk, unsigned* __restrict__ status)
{
    const StageLayout L(H, topk);
    const int p = blockIdx.x, tid = threadIdx.x;
    char* dst = a.stage[p];
    char* own = a.stage[a.rank];
    unsigned* ctl = (unsigned*) (own + L.ctl);                     // [0] step number, [1] finished blocks of this launch
    const unsigned g = *(volatile unsigned*) ctl + 1u;            // advanced only after every block of this launch has read it
    const int n_own = R > a.rank ? (R - a.rank + a.world - 1) / a.world : 0;
    const int words = H / 8;                                       // 16-byte words per row
    // all of a thread's loads are issued before its first store: the copy costs one load latency, not one per word
    constexpr int U = 8;
    for (int base = tid; base < n_own * words; base += DISPATCH_THREADS * U)
    {
        uint4 v[U];
        #pragma unroll
        for (int u = 0; u < U; ++u) { const int i = base + u * DISPATCH_THREADS; if (i < n_own * words) v[u] = x_own[i]; }
        #pragma unroll
        for (int u = 0; u < U; ++u)
        {
            const int i = base + u * DISPATCH_THREADS;
            if (i < n_own * words) { const int j = i / words, c = i - j * words; ((uint4*) (dst + L.x))[(size_t) (a.rank + j * a.world) * words + c] = v[u]; }
        }
    }
    for (int i = tid; i < n_own * topk; i += blockDim.x)
    {
        const int j = i / topk, k = i - j * topk, r = a.rank + j * a.world;
        ((int64_t*) (dst + L.sel))[r * topk + k] = sel_own[i];
        ((uint16_t*) (dst + L.rw))[r * topk + k] = rw_own[i];
    }
    __syncthreads();
    if (tid == 0)
    {
        __threadfence_system();
        st_release_sys((unsigned*) (dst + L.flags) + a.rank, g);
        const unsigned long long t0 = globaltimer_ns();
        while ((int) (ld_acquire_sys((const unsigned*) (own + L.flags) + p) - g) < 0)
            if (globaltimer_ns() - t0 > 2000000000ull) { atomicOr(status, ST_WAIT_TIMEOUT); break; }
        __threadfence();
        if (atomicAdd(ctl + 1, 1u) == gridDim.x - 1) { ctl[1] = 0u; *(volatile unsigned*) ctl = g; }
    }
}

// Prefill dispatch as an all-to-all-v over peer memory: one warp per row of the rank's slice. The row goes, at its global position,
// into the staging area of every rank that holds one of its selected experts (position e belongs to rank e / n_per_rank) and into
// the rank's own (the shared expert runs where the row lives); the selections and weights go to every rank (a row costs 80 bytes
// there, 12 KB here). A rank that does not need a row keeps whatever its staging area held at that position and never reads it:
// its permutation only lists rows with a local expert. The flag barrier that follows (ep_barrier_kernel, next launch of the stream)
// publishes the stores.
struct PrefillStage
{
    size_t sel, rw, total;          // x at 0: [R][H] 16-bit; sel int64 [R][topk]; rw 16-bit [R][topk]
    __host__ __device__ PrefillStage(int R, int H, int topk)
    {
        sel = ((size_t) R * H * 2 + 255) / 256 * 256;
        rw = sel + ((size_t) R * topk * 8 + 255) / 256 * 256;
        total = rw + ((size_t) R * topk * 2 + 255) / 256 * 256;
    }
};

__global__ void __launch_bounds__(256) prefill_dispatch_kernel(const StageArgs a, const uint4* __restrict__ x_own, const int64_t* __restrict__ sel_own,
                                                               const uint16_t* __restrict__ rw_own, int rpr, int H, int topk, int n_per_rank,
                                                               unsigned long long* __restrict__ sent_rows)
{
    const PrefillStage L(rpr * a.world, H, topk);
    const int lane = threadIdx.x & 31, warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = (gridDim.x * blockDim.x) >> 5;
    const int words = H / 8;
    unsigned long long sent = 0;
    for (int row = warp; row < rpr; row += nwarps)
    {
        const size_t grow = (size_t) a.rank * rpr + row;
        unsigned m = 0;
        if (lane < topk)
        {
            const int64_t e = sel_own[(size_t) row * topk + lane];
            const uint16_t w = rw_own[(size_t) row * topk + lane];
            if (e >= 0 && e < (int64_t) a.world * n_per_rank) m = 1u << (int) (e / n_per_rank);
            for (int p = 0; p < a.world; ++p)
            {
                ((int64_t*) (a.stage[p] + L.sel))[grow * topk + lane] = e;
                ((uint16_t*) (a.stage[p] + L.rw))[grow * topk + lane] = w;
            }
        }
        m = __reduce_or_sync(0xffffffffu, m) | (1u << a.rank);
        sent += __popc(m & ~(1u << a.rank));
        const uint4* src = x_own + (size_t) row * words;
        constexpr int U = 4;                       // a lane's loads of a pass are issued before its first store
        for (int c0 = lane; c0 < words; c0 += 32 * U)
        {
            uint4 v[U];
            #pragma unroll
            for (int u = 0; u < U; ++u) if (c0 + 32 * u < words) v[u] = src[c0 + 32 * u];
            for (int p = 0; p < a.world; ++p)
            {
                if (!((m >> p) & 1u)) continue;
                uint4* dst = (uint4*) a.stage[p] + grow * words;
                #pragma unroll
                for (int u = 0; u < U; ++u) if (c0 + 32 * u < words) dst[c0 + 32 * u] = v[u];
            }
        }
    }
    if (sent_rows && lane == 0 && sent) atomicAdd(sent_rows, sent);
}

// Barrier over the ranks through the same flags: raise generation `gen` in every peer's memory, wait (bounded) until every
// peer has raised it here. What a rank wrote into peer memory before this kernel (in stream order) is complete when the
// peers pass the barrier: the flag is stored with release semantics at system scope after a system-wide fence.
__global__ void __launch_bounds__(32) ep_barrier_kernel(const EpArgs a, unsigned gen, unsigned* __restrict__ status)
{
    __threadfence_system();
    if ((int) threadIdx.x < a.world) st_release_sys(a.flags[threadIdx.x] + a.rank, gen);
    if ((int) threadIdx.x < a.world)
    {
        const unsigned long long t0 = globaltimer_ns();
        while ((int) (ld_acquire_sys(a.flags[a.rank] + threadIdx.x) - gen) < 0)
            if (globaltimer_ns() - t0 > 2000000000ull) { atomicOr(status, ST_WAIT_TIMEOUT); break; }
    }
    __threadfence_system();
}

}  // namespace

int ep_barrier_launch(int rank, int world, void* const* flags, unsigned gen, unsigned* status, cudaStream_t st)
{
    if (world < 1 || world > 8 || rank < 0 || rank >= world || !flags || !status) return fail(HMOE_E_ARG, "hmoe_ep_barrier: arguments");
    EpArgs a;
    a.rank = rank; a.world = world;
    for (int p = 0; p < 8; ++p) { a.slots[p] = nullptr; a.flags[p] = p < world ? (unsigned*) flags[p] : nullptr; }
    ep_barrier_kernel<<<1, 32, 0, st>>>(a, gen, status);
    count_launches(1);
    const cudaError_t err = cudaGetLastError();
    return err == cudaSuccess ? HMOE_OK : fail(HMOE_E_CUDA, cudaGetErrorString(err));
}

size_t ep_stage_bytes(int H, int topk) { return StageLayout(H, topk).total; }

int ep_dispatch_launch(int rank, int world, void* const* stage, const void* x_own, const int64_t* sel_own, const void* rw_own, int R, int H, int topk,
                       unsigned* status, cudaStream_t st)
{
    if (world < 1 || world > 8 || rank < 0 || rank >= world) return fail(HMOE_E_ARG, "hmoe_ep_dispatch: world must be 1..8");
    if (!stage || !status || R < 1 || R > MAXR || H % 8 || topk < 1 || topk > TOPK_MAX) return fail(HMOE_E_ARG, "hmoe_ep_dispatch: rows 1..16, H % 8 == 0, topk 1..8");
    if (R > rank && (!x_own || !sel_own || !rw_own)) return fail(HMOE_E_ARG, "hmoe_ep_dispatch: null pointer");
    StageArgs a;
    a.rank = rank; a.world = world;
    for (int p = 0; p < 8; ++p) a.stage[p] = p < world ? (char*) stage[p] : nullptr;
    ep_dispatch_kernel<<<world, DISPATCH_THREADS, 0, st>>>(a, (const uint4*) x_own, sel_own, (const uint16_t*) rw_own, R, H, topk, status);
    count_launches(1);
    const cudaError_t err = cudaGetLastError();
    return err == cudaSuccess ? HMOE_OK : fail(HMOE_E_CUDA, cudaGetErrorString(err));
}

int ep_combine_launch(int rank, int world, void* const* slots, void* const* flags, const unsigned* gen, float* f, int rows, int H, size_t slot_floats,
                      unsigned* status, cudaStream_t st, int own_rows)
{
    if (world < 1 || world > 8 || rank < 0 || rank >= world) return fail(HMOE_E_ARG, "hmoe_ep_combine: world must be 1..8");
    const int n = rows * H;
    if (!f || !slots || !flags || !status || !gen || n <= 0 || n % 4 || (size_t) n > slot_floats) return fail(HMOE_E_ARG, "hmoe_ep_combine: sizes");
    EpArgs a;
    a.rank = rank; a.world = world;
    for (int p = 0; p < 8; ++p) { a.slots[p] = p < world ? (float*) slots[p] : nullptr; a.flags[p] = p < world ? (unsigned*) flags[p] : nullptr; }
    const int blocks = (n / 4 + 255) / 256 < 96 ? (n / 4 + 255) / 256 : 96;
    if (H % 4) return fail(HMOE_E_ARG, "hmoe_ep_combine: H must be a multiple of 4");
    {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(blocks); cfg.blockDim = dim3(256); cfg.stream = st;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at; cfg.numAttrs = 1;
        cudaLaunchKernelEx(&cfg, ep_combine_kernel, a, gen, f, n, slot_floats, status, own_rows, H);
    }
    count_launches(1);
    const cudaError_t err = cudaGetLastError();
    return err == cudaSuccess ? HMOE_OK : fail(HMOE_E_CUDA, cudaGetErrorString(err));
}

size_t prefill_stage_bytes(int R, int H, int topk) { return PrefillStage(R, H, topk).total; }
void prefill_stage_offsets(int R, int H, int topk, size_t* sel_off, size_t* rw_off) { const PrefillStage L(R, H, topk); *sel_off = L.sel; *rw_off = L.rw; }

int prefill_dispatch_launch(int rank, int world, void* const* stage, const void* x_own, const int64_t* sel_own, const void* rw_own, int rpr, int H,
                            int topk, int n_per_rank, unsigned long long* sent_rows, cudaStream_t st)
{
    if (world < 1 || world > 8 || rank < 0 || rank >= world) return fail(HMOE_E_ARG, "hmoe_prefill_ep_dispatch: world must be 1..8");
    if (!stage || !x_own || !sel_own || !rw_own || rpr < 1 || H % 8 || topk < 1 || topk > 32 || n_per_rank < 1)
        return fail(HMOE_E_ARG, "hmoe_prefill_ep_dispatch: arguments");
    StageArgs a;
    a.rank = rank; a.world = world;
    for (int p = 0; p < 8; ++p) a.stage[p] = p < world ? (char*) stage[p] : nullptr;
    const int blocks = 2 * device_sms();
    prefill_dispatch_kernel<<<blocks, 256, 0, st>>>(a, (const uint4*) x_own, sel_own, (const uint16_t*) rw_own, rpr, H, topk, n_per_rank, sent_rows);
    count_launches(1);
    const cudaError_t err = cudaGetLastError();
    return err == cudaSuccess ? HMOE_OK : fail(HMOE_E_CUDA, cudaGetErrorString(err));
}

}  // namespace hmoe

using namespace hmoe;

extern "C" {

int hmoe_ep_alloc(size_t bytes, void** ptr)
{
    if (!ptr || bytes == 0) return fail(HMOE_E_ARG, "hmoe_ep_alloc: arguments");
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e == cudaSuccess) e = cudaMemset(p, 0, bytes);
    if (e != cudaSuccess) return fail(HMOE_E_CUDA, cudaGetErrorString(e));
    *ptr = p;
    return HMOE_OK;
}
int hmoe_ep_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? HMOE_OK : fail(HMOE_E_CUDA, "hmoe_ep_free: cudaFree failed"); }
int hmoe_ep_export(void* ptr, unsigned char* handle64)
{
    if (!ptr || !handle64) return fail(HMOE_E_ARG, "hmoe_ep_export: arguments");
    cudaIpcMemHandle_t h;
    const cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
    if (e != cudaSuccess) return fail(HMOE_E_CUDA, cudaGetErrorString(e));
    static_assert(sizeof(h) == 64, "ipc handle size");
    memcpy(handle64, &h, 64);
    return HMOE_OK;
}
int hmoe_ep_open(const unsigned char* handle64, void** ptr)
{
    if (!ptr || !handle64) return fail(HMOE_E_ARG, "hmoe_ep_open: arguments");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void* p = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return fail(HMOE_E_CUDA, cudaGetErrorString(e));
    *ptr = p;
    return HMOE_OK;
}
int hmoe_ep_close(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? HMOE_OK : fail(HMOE_E_CUDA, "hmoe_ep_close failed"); }

int hmoe_ep_combine(int rank, int world, void* const* slots, void* const* flags, const uint32_t* gen, float* f, int rows, int H, size_t slot_floats,
                    uint32_t* status, void* stream)
{
    return ep_combine_launch(rank, world, slots, flags, gen, f, rows, H, slot_floats, status, (cudaStream_t) stream, 0);
}

int hmoe_ep_combine_own(int rank, int world, void* const* slots, void* const* flags, const uint32_t* gen, float* f_own, int rows, int H,
                        size_t slot_floats, uint32_t* status, void* stream)
{
    return ep_combine_launch(rank, world, slots, flags, gen, f_own, rows, H, slot_floats, status, (cudaStream_t) stream, 1);
}

size_t hmoe_ep_stage_bytes(int H, int topk) { return ep_stage_bytes(H, topk); }
int hmoe_ep_stage_offsets(int H, int topk, size_t* x_off, size_t* sel_off, size_t* rw_off)
{
    if (!x_off || !sel_off || !rw_off) return fail(HMOE_E_ARG, "hmoe_ep_stage_offsets: null pointer");
    const StageLayout L(H, topk);
    *x_off = L.x; *sel_off = L.sel; *rw_off = L.rw;
    return HMOE_OK;
}
int hmoe_ep_dispatch(int rank, int world, void* const* stage, const void* x_own, const int64_t* sel_own, const void* rw_own, int R, int H, int topk,
                     uint32_t* status, void* stream)
{
    return ep_dispatch_launch(rank, world, stage, x_own, sel_own, rw_own, R, H, topk, status, (cudaStream_t) stream);
}

int hmoe_ep_memset(void* ptr, int value, size_t bytes, void* stream)
{
    if (!ptr) return fail(HMOE_E_ARG, "hmoe_ep_memset: null pointer");
    return cudaMemsetAsync(ptr, value, bytes, (cudaStream_t) stream) == cudaSuccess ? HMOE_OK : fail(HMOE_E_CUDA, "hmoe_ep_memset: cudaMemsetAsync failed");
}
int hmoe_ep_copy(void* dst, const void* src, size_t bytes, void* stream)
{
    if (!dst || !src) return fail(HMOE_E_ARG, "hmoe_ep_copy: null pointer");
    return cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t) stream) == cudaSuccess ? HMOE_OK
                                                                                                           : fail(HMOE_E_CUDA, "hmoe_ep_copy: cudaMemcpyAsync failed");
}

int hmoe_ep_barrier(int rank, int world, void* const* flags, uint32_t gen, uint32_t* status, void* stream)
{
    return ep_barrier_launch(rank, world, flags, gen, status, (cudaStream_t) stream);
}

size_t hmoe_prefill_ep_stage_bytes(int rows_total, int H, int topk) { return prefill_stage_bytes(rows_total, H, topk); }
int hmoe_prefill_ep_stage_offsets(int rows_total, int H, int topk, size_t* sel_off, size_t* rw_off)
{
    if (!sel_off || !rw_off) return fail(HMOE_E_ARG, "hmoe_prefill_ep_stage_offsets: null pointer");
    prefill_stage_offsets(rows_total, H, topk, sel_off, rw_off);
    return HMOE_OK;
}
int hmoe_prefill_ep_dispatch(int rank, int world, void* const* stage, const void* x_own, const int64_t* sel_own, const void* rw_own, int rows_per_rank,
                             int H, int topk, int n_per_rank, unsigned long long* sent_rows, void* stream)
{
    return prefill_dispatch_launch(rank, world, stage, x_own, sel_own, rw_own, rows_per_rank, H, topk, n_per_rank, sent_rows, (cudaStream_t) stream);
}

}  // extern "C"

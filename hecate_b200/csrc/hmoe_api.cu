// The C ABI of libhecate_moe_b200.so (declared in include/hecate_moe.h) and the small stand-alone kernels: combine,
// dequantise, status readback and the synthetic-data fill.
#include <atomic>
#include <cstdio>
#include <cstring>
#include "hmoe_common.cuh"
#include "hmoe_internal.h"
#include "hmoe_prepare.cuh"

namespace hmoe {

static thread_local char g_err[256] = "";
static std::atomic<int64_t> g_launches{0};

int fail(int code, const char* msg)
{
    snprintf(g_err, sizeof(g_err), "%s", msg ? msg : "");
    return code;
}
void count_launches(int n) { g_launches += n; }

int current_device()
{
    int d = -1;
    return cudaGetDevice(&d) == cudaSuccess ? d : -1;
}
int device_sms()
{
    static std::atomic<int> sms[MAX_DEVICES] = {};
    const int d = current_device();
    if (d < 0) return 0;
    if (d < MAX_DEVICES) { const int v = sms[d].load(std::memory_order_relaxed); if (v) return v; }
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, d) != cudaSuccess) return 0;
    if (d < MAX_DEVICES) sms[d].store(n, std::memory_order_relaxed);
    return n;
}

namespace {

// f += y (+ o) (+ o2), y = 0: the band partials are added in the reference's fixed order ((f + y) + o) + o2
// (runtime/tier/moe4/moe4.cu:702-717; runtime/tier/cn.cu:3)
__global__ void __launch_bounds__(256) combine_kernel(float* __restrict__ f, const float* __restrict__ o, float* __restrict__ y,
                                                      int64_t n, const float* __restrict__ o2)
{
    // launched with programmatic stream serialization: the blocks may be resident before the kernel that produced y has finished
    asm volatile("griddepcontrol.wait;" ::: "memory");
    TL_MIN(0);
    const int64_t i = ((int64_t) blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= n) return;
    float4 a = *(float4*) (f + i);
    const float4 c = *(const float4*) (y + i);
    a.x += c.x; a.y += c.y; a.z += c.z; a.w += c.w;
    if (o) { const float4 b = *(const float4*) (o + i); a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w; }
    if (o2) { const float4 b = *(const float4*) (o2 + i); a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w; }
    *(float4*) (f + i) = a;
    *(float4*) (y + i) = make_float4(0.f, 0.f, 0.f, 0.f);
}

// Ordered sum of partial outputs + residual add + RMS norm, one launch (replaces combine_norm, runtime/tier/cn.cu:50-105, and is
// also the tail of the expert-parallel combine). One block of 1024 threads per row. The list `part` holds the row-major fp32
// partials in the order they are added (the reference's order is ((f + y) + o) + o2; a null first entry reads as zero); `clear`
// (the accumulator the expert kernels add into) is zeroed for the next layer. What the bit-identity contract with the
// reference kernel fixes is arithmetic only: thread t owns 4-wide columns t, t + 1024, ..., squares are accumulated with fused
// multiply-adds in element order, the 1024 partial sums are reduced by a butterfly inside each warp and a second butterfly over
// the 32 warp sums, and xn = fp16((r * (w + cbias)) * (rsqrt(mean + eps) * cscale)).
constexpr int NORM_THREADS = 1024, NORM_VECS = 4, NORM_PARTS = 10;

struct NormParts
{
    const float* part[NORM_PARTS];     // added in this order; part[0] may be null (= zeros), the others are all valid
    int n;
    float* clear;                      // zeroed after it was read (may be null)
};

template <bool WBF>
__global__ void __launch_bounds__(NORM_THREADS) sum_norm_kernel(const NormParts in, float* __restrict__ resid, const uint16_t* __restrict__ w,
                                                                __half* __restrict__ xn, int H, float eps, float cbias, float cscale)
{
    __shared__ float warp_sum[32];
    const int tid = threadIdx.x, nvec = H / 4;
    const size_t row = (size_t) blockIdx.x * H;
    float4 keep[NORM_VECS];
    float ss = 0.f;
    #pragma unroll
    for (int j = 0; j < NORM_VECS; ++j)
    {
        const int vec = tid + j * NORM_THREADS;
        if (vec < nvec)
        {
            const size_t at = row + 4 * (size_t) vec;
            float4 sum = in.part[0] ? *(const float4*) (in.part[0] + at) : make_float4(0.f, 0.f, 0.f, 0.f);
            for (int p = 1; p < in.n; ++p) sum = vec_add(sum, *(const float4*) (in.part[p] + at));
            sum = vec_add(sum, *(const float4*) (resid + at));
            if (in.clear) *(float4*) (in.clear + at) = make_float4(0.f, 0.f, 0.f, 0.f);
            *(float4*) (resid + at) = sum;
            keep[j] = sum;
            ss = sq_accumulate(ss, sum);
        }
    }
    ss = butterfly32(ss);
    if ((tid & 31) == 0) warp_sum[tid >> 5] = ss;
    __syncthreads();
    const float total = butterfly32(warp_sum[tid & 31]);
    const float k = rsqrtf(total / (float) H + eps) * cscale;
    #pragma unroll
    for (int j = 0; j < NORM_VECS; ++j)
    {
        const int vec = tid + j * NORM_THREADS;
        if (vec < nvec) *(uint2*) (xn + row + 4 * (size_t) vec) = norm_pack4(keep[j], norm_weight4<WBF>(w, vec), cbias, k);
    }
}

// one thread per 16-byte word of packed codes: 4 x 8 codes -> fp16 [N][K] times the scale of (row, column group)
__global__ void __launch_bounds__(256) dequant_kernel(const uint4* __restrict__ q, const void* __restrict__ sc, int group, int N, int K,
                                                      __half* __restrict__ out)
{
    const int KB = K / 64;
    const size_t total = (size_t) N / 16 * KB * 32;
    for (size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t) gridDim.x * blockDim.x)
    {
        const int lane = (int) (i & 31), s = (int) ((i >> 5) & 3), kb = (int) ((i >> 7) % KB), gr = (int) ((i >> 7) / KB);
        const int g = lane >> 2, qq = lane & 3;
        const uint4 v = q[i];
        const uint32_t ww[4] = {v.x, v.y, v.z, v.w};
        #pragma unroll
        for (int t = 0; t < 4; ++t)
            #pragma unroll
            for (int nib = 0; nib < 8; ++nib)
            {
                const int cc = nib >> 2, h = (nib >> 1) & 1, rh = nib & 1;
                const int row = gr * 64 + s * 16 + rh * 8 + g, k = kb * 64 + t * 16 + h * 8 + qq * 2 + cc;
                const float scale = group ? bf16_bits_to_float(((const uint16_t*) sc)[((size_t) (row >> 6) * (K / group) + k / group) * 64 + (row & 7) * 8 + ((row & 63) >> 3)])
                                          : ((const float*) sc)[row];
                out[(size_t) row * K + k] = __float2half_rn((float) ((int) ((ww[t] >> (4 * nib)) & 15) - 8) * scale);
            }
    }
}

__device__ __forceinline__ unsigned long long mix64(unsigned long long z)
{
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__global__ void __launch_bounds__(256) fill_kernel(unsigned long long* __restrict__ dst, size_t nwords, unsigned long long base)
{
    for (size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x; i < nwords; i += (size_t) gridDim.x * blockDim.x)
        dst[i] = mix64(base + i);
}

}  // namespace
}  // namespace hmoe

using namespace hmoe;

extern "C" {

int hmoe_version(void) { return 100; }
const char* hmoe_last_error(void) { return g_err; }
int64_t hmoe_launch_count(void) { return g_launches.load(); }

size_t hmoe_router_ws_bytes(int R, int E) { return router_ws_bytes(R, E); }
int hmoe_router(const void* x, int x_dtype, const void* wt, int w_dtype, const float* bias, int R, int H, int E, int topk,
                float scale, int64_t* sel, void* rw, void* ws, size_t ws_bytes, void* stream)
{
    return router_launch(x, x_dtype, wt, w_dtype, bias, R, H, E, topk, scale, sel, rw, ws, ws_bytes, (cudaStream_t) stream);
}

int hmoe_norm_router(const float* y, const float* r, float* r_out, const void* nw, int nw_dtype, void* xn, const void* wt, int w_dtype,
                     const float* bias, int R, int H, int E, int topk, float scale, float eps, float cbias, float cscale, int64_t* sel, void* rw,
                     void* ws, size_t ws_bytes, void* stream)
{
    return norm_router_launch(y, r, r_out, nw, nw_dtype, xn, wt, w_dtype, bias, R, H, E, topk, scale, eps, cbias, cscale, sel, rw, ws, ws_bytes,
                              (cudaStream_t) stream);
}

size_t hmoe_decode_ws_bytes(int H, int I) { return decode_ws_bytes(H, I); }
int hmoe_decode(const hmoe_layer* layer, const void* x, int x_dtype, const int64_t* sel, const void* rw, int R, int lo, int n_local,
                int act_quant, float* y, void* ws, size_t ws_bytes, void* stream)
{
    if (!layer) return fail(HMOE_E_ARG, "hmoe_decode: null layer");
    return decode_launch(layer, x, x_dtype, sel, rw, R, lo, n_local, act_quant, y, ws, ws_bytes, (cudaStream_t) stream);
}

int hmoe_router_decode(const hmoe_layer* layer, const void* x, int x_dtype, const void* wt, int w_dtype, const float* bias, int R, int E, float scale,
                       int64_t* sel, void* rw, void* router_ws, size_t router_ws_bytes, int lo, int n_local, int act_quant, float* y, void* ws,
                       size_t ws_bytes, void* stream)
{
    if (!layer) return fail(HMOE_E_ARG, "hmoe_router_decode: null layer");
    PrepArgs pa;
    int rc = decode_prep_args(layer, x, x_dtype, R, lo, n_local, act_quant, ws, ws_bytes, 1, 0, nullptr, &pa);
    if (rc) return rc;
    rc = router_prepare_launch(x, x_dtype, wt, w_dtype, bias, R, layer->H, E, layer->topk, scale, sel, rw, router_ws, router_ws_bytes, pa, (cudaStream_t) stream);
    if (rc) return rc;
    return decode_launch(layer, x, x_dtype, sel, rw, R, lo, n_local, act_quant, y, ws, ws_bytes, (cudaStream_t) stream, 1, 0, nullptr, 0, true);
}

size_t hmoe_prefill_ws_bytes(int R, int topk, int n_local, int H, int I, int act_quant) { return prefill_ws_bytes(R, topk, n_local, H, I, act_quant); }
int hmoe_prefill(const hmoe_layer* layer, const void* x, int x_dtype, const int64_t* sel, const void* rw, int R, int lo, int n_local,
                 int act_quant, float* out, void* ws, size_t ws_bytes, void* stream)
{
    if (!layer) return fail(HMOE_E_ARG, "hmoe_prefill: null layer");
    return prefill_launch(layer, x, x_dtype, sel, rw, R, lo, n_local, act_quant, out, ws, ws_bytes, (cudaStream_t) stream);
}
size_t hmoe_short_prefill_ws_bytes(int R, int H, int I, int topk) { return R < 1 || R > SHORT_MAXR || topk < 1 || topk > TOPK_MAX ? 0 : short_ws_bytes(R, H, I, topk); }
int hmoe_short_prefill(const hmoe_layer* layer, const void* x, int x_dtype, const int64_t* sel, const void* rw, int R, int lo, int n_local,
                       int act_quant, float* out, void* ws, size_t ws_bytes, void* stream)
{
    if (!layer) return fail(HMOE_E_ARG, "hmoe_short_prefill: null layer");
    return short_launch(layer, x, x_dtype, sel, rw, R, lo, n_local, act_quant, out, ws, ws_bytes, (cudaStream_t) stream);
}

int hmoe_short_prefill_ep(const hmoe_layer* layer, const void* x, int x_dtype, const int64_t* sel, const void* rw, int R, int lo, int n_local,
                          int act_quant, float* out, void* ws, size_t ws_bytes, int shared_row0, int shared_rows, void* stream)
{
    if (!layer) return fail(HMOE_E_ARG, "hmoe_short_prefill_ep: null layer");
    if (shared_rows < 0) return fail(HMOE_E_ARG, "hmoe_short_prefill_ep: shared_rows must be >= 0");
    return short_launch(layer, x, x_dtype, sel, rw, R, lo, n_local, act_quant, out, ws, ws_bytes, (cudaStream_t) stream, shared_row0, shared_rows);
}

// Which path serves a call of R rows: 0 decode, 1 short prefill, 2 grouped GEMMs. The short path needs the shapes whose tile
// activations fit in registers; FORWARD_SHORT_ROWS is where the grouped GEMMs become faster
// (measured on the benchmark layer: they cost the same from about 100 rows up because every expert's weights are converted
// whatever its row count, the short path grows with the number of 8-pick tiles).
static int forward_path(const hmoe_layer* L, int R, int act_quant)
{
    const bool sh8 = L->shared_format == 1 && L->sh_gate_w != nullptr;
    if (sh8 && act_quant) return 2;           // the int8 shared expert in the int8 activation mode: only the grouped GEMMs serve it
    if (R <= MAXR) return 0;
    // the int8 shared expert costs the short path two small launches per sixteen rows (0.43 ms at 256 rows): it hands over earlier
    if (R <= (sh8 ? FORWARD_SHORT_ROWS_SH8 : FORWARD_SHORT_ROWS) && L->I <= 2048 && L->H <= 6144) return 1;
    return 2;
}
int hmoe_forward_short_rows(void) { return FORWARD_SHORT_ROWS; }
size_t hmoe_forward_ws_bytes(int R, int topk, int n_local, int H, int I, int act_quant)
{
    if (R < 1 || topk < 1 || topk > TOPK_MAX) return 0;
    size_t b = decode_ws_bytes(H, I);
    const int rs = R < FORWARD_SHORT_ROWS ? R : FORWARD_SHORT_ROWS;
    if (R > MAXR) { const size_t s = short_ws_bytes(rs, H, I, topk); b = s > b ? s : b; }
    { const size_t p = prefill_ws_bytes(R, topk, n_local, H, I, act_quant); b = p > b ? p : b; }      // any R can end up there (see forward_path)
    return b;
}
int hmoe_forward(const hmoe_layer* layer, const void* x, int x_dtype, const int64_t* sel, const void* rw, int R, int lo, int n_local,
                 int act_quant, float* out, void* ws, size_t ws_bytes, void* stream)
{
    if (!layer) return fail(HMOE_E_ARG, "hmoe_forward: null layer");
    if (R < 1) return fail(HMOE_E_ARG, "hmoe_forward: rows must be >= 1");
    if (ws_bytes < hmoe_forward_ws_bytes(R, layer->topk, n_local, layer->H, layer->I, act_quant)) return fail(HMOE_E_WS, "hmoe_forward: workspace too small");
    switch (forward_path(layer, R, act_quant))
    {
    case 0: return decode_launch(layer, x, x_dtype, sel, rw, R, lo, n_local, act_quant, out, ws, ws_bytes, (cudaStream_t) stream);
    case 1: return short_launch(layer, x, x_dtype, sel, rw, R, lo, n_local, act_quant, out, ws, ws_bytes, (cudaStream_t) stream);
    default: return prefill_launch(layer, x, x_dtype, sel, rw, R, lo, n_local, act_quant, out, ws, ws_bytes, (cudaStream_t) stream);
    }
}
int hmoe_prefill_ep(const hmoe_layer* layer, const void* x, int x_dtype, const int64_t* sel, const void* rw, int R, int lo, int n_local,
                    int act_quant, float* out, void* ws, size_t ws_bytes, int shared_row0, int shared_rows, void* stream)
{
    if (!layer) return fail(HMOE_E_ARG, "hmoe_prefill_ep: null layer");
    if (shared_rows < 0) return fail(HMOE_E_ARG, "hmoe_prefill_ep: shared_rows must be >= 0");
    return prefill_launch(layer, x, x_dtype, sel, rw, R, lo, n_local, act_quant, out, ws, ws_bytes, (cudaStream_t) stream, shared_row0, shared_rows);
}
int hmoe_prefill_ep_peer(const hmoe_layer* layer, const void* x, int x_dtype, const int64_t* sel, const void* rw, int R, int lo, int n_local,
                         int act_quant, void* const* out_peer, int world, int rows_per_rank, void* ws, size_t ws_bytes, int shared_row0,
                         int shared_rows, void* stream)
{
    if (!layer) return fail(HMOE_E_ARG, "hmoe_prefill_ep_peer: null layer");
    if (!out_peer) return fail(HMOE_E_ARG, "hmoe_prefill_ep_peer: null output table");
    return prefill_launch(layer, x, x_dtype, sel, rw, R, lo, n_local, act_quant, nullptr, ws, ws_bytes, (cudaStream_t) stream, shared_row0, shared_rows,
                          out_peer, world, rows_per_rank);
}

size_t hmoe_prefill_sorted_ws_bytes(int npos, int H, int I, int act_quant) { return prefill_sorted_ws_bytes(npos, H, I, act_quant); }
int hmoe_prefill_sorted(const hmoe_layer* layer, const void* x, int x_dtype, const int32_t* tok, const float* wt, const int32_t* rbt, int nrb,
                        int npos, int n_local, int act_quant, float* out, void* ws, size_t ws_bytes, void* stream)
{
    if (!layer) return fail(HMOE_E_ARG, "hmoe_prefill_sorted: null layer");
    return prefill_sorted_launch(layer, x, x_dtype, tok, wt, rbt, nrb, npos, n_local, act_quant, out, ws, ws_bytes, (cudaStream_t) stream);
}
size_t hmoe_permute_ws_bytes(int R, int topk, int n_local) { return permute_ws_bytes(R, topk, n_local); }
int hmoe_permute(const int64_t* sel, const void* rw, int R, int topk, int lo, int n_local, int shared_rows, int bm, int balance,
                 int32_t* order, int32_t* tok, int32_t* eid, float* wt, int32_t* counts, int32_t* rbt, int32_t* plan, void* ws, size_t ws_bytes,
                 void* stream)
{
    return permute_launch(sel, rw, R, topk, lo, n_local, shared_rows, bm, balance, order, tok, eid, wt, counts, rbt, plan, ws, ws_bytes,
                          (cudaStream_t) stream);
}

int hmoe_set_profiling(int on) { return decode_set_profiling(on); }
int hmoe_decode_phase_times(float* ms3) { return ms3 ? decode_phase_times(ms3) : fail(HMOE_E_ARG, "hmoe_decode_phase_times: null pointer"); }

int hmoe_decode_ep(const hmoe_layer* layer, const void* x, int x_dtype, const int64_t* sel, const void* rw, int R, int lo, int n_local,
                   int act_quant, float* y, void* ws, size_t ws_bytes, int shared_mod, int shared_rem, uint32_t* gen, size_t slot_floats,
                   void* stream)
{
    if (!layer) return fail(HMOE_E_ARG, "hmoe_decode_ep: null layer");
    return decode_launch(layer, x, x_dtype, sel, rw, R, lo, n_local, act_quant, y, ws, ws_bytes, (cudaStream_t) stream, shared_mod, shared_rem,
                         gen, slot_floats);
}

int hmoe_decode_ep_combine(const hmoe_layer* layer, const void* x, int x_dtype, const int64_t* sel, const void* rw, int R, int lo, int n_local,
                           int act_quant, void* ws, size_t ws_bytes, int shared_mod, int shared_rem, uint32_t* gen, size_t slot_floats, int rank,
                           int world, void* const* slots, void* const* flags, float* f, int own_rows, uint32_t* status, void* stream)
{
    if (!layer) return fail(HMOE_E_ARG, "hmoe_decode_ep_combine: null layer");
    if (!slots || rank < 0 || rank >= world || world > 8) return fail(HMOE_E_ARG, "hmoe_decode_ep_combine: rank / world / slots");
    EpCombineArgs e = {rank, world, own_rows, slots, flags, f, status};
    return decode_launch(layer, x, x_dtype, sel, rw, R, lo, n_local, act_quant, (float*) slots[rank], ws, ws_bytes, (cudaStream_t) stream, shared_mod,
                         shared_rem, gen, slot_floats, false, &e);
}

int hmoe_decode_ep_dp(const hmoe_layer* layer, const void* x_own, int x_dtype, const void* wt, int w_dtype, const float* bias, int R, int E,
                      float scale, int64_t* sel, void* rw, void* router_ws, size_t router_ws_bytes, int lo, int n_local, int act_quant, void* ws,
                      size_t ws_bytes, int rank, int world, void* const* stage, void* const* slots, void* const* flags, uint32_t* gen,
                      size_t slot_floats, float* f_own, uint32_t* status, int fused_tail, void* stream)
{
    if (!layer) return fail(HMOE_E_ARG, "hmoe_decode_ep_dp: null layer");
    if (world < 1 || world > 8 || rank < 0 || rank >= world || !stage || !slots || !flags || !gen || !status || !f_own)
        return fail(HMOE_E_ARG, "hmoe_decode_ep_dp: world 1..8, buffers");
    if (R < 1 || R > MAXR || layer->H % 8) return fail(HMOE_E_ARG, "hmoe_decode_ep_dp: rows 1..16");
    const int n_own = R > rank ? (R - rank + world - 1) / world : 0;
    if (n_own > 0 && !x_own) return fail(HMOE_E_ARG, "hmoe_decode_ep_dp: null rows");
    const StageLayout SL(layer->H, layer->topk);
    const void* x_all = (const char*) stage[rank] + SL.x;          // after the launch below: all rows, in the local staging area
    PrepArgs pa;
    int rc = decode_prep_args(layer, x_all, x_dtype, R, lo, n_local, act_quant, ws, ws_bytes, world, rank, gen, &pa);
    if (rc) return rc;
    if (world > 1 && E % world == 0 && n_local == 2 * (E / world))
    {
        // every expert on two ranks: this rank's tables hold the bands rank and rank + 1 (mod world) of E / world router positions
        if (E > 256 || lo != rank * (E / world)) return fail(HMOE_E_ARG, "hmoe_decode_ep_dp: two bands per rank need lo = rank * E / world and E <= 256");
        pa.n_total = E; pa.bal_world = world; pa.bal_rank = rank;
    }
    DispArgs da;
    da.rank = rank; da.world = world; da.n_own = n_own; da.words = layer->H / 8; da.x_own = (const uint4*) x_own;
    da.x_off = SL.x; da.flags_off = SL.flags; da.ctl_off = SL.ctl;
    for (int p = 0; p < 8; ++p) da.stage[p] = p < world ? (char*) stage[p] : nullptr;
    cudaStream_t st = (cudaStream_t) stream;
    rc = router_prepare_launch(x_all, x_dtype, wt, w_dtype, bias, R, layer->H, E, layer->topk, scale, sel, rw, router_ws, router_ws_bytes, pa, st, &da);
    if (rc) return rc;
    EpCombineArgs e = {rank, world, 1, slots, flags, f_own, status};
    rc = decode_launch(layer, x_all, x_dtype, sel, rw, R, lo, n_local, act_quant, (float*) slots[rank], ws, ws_bytes, st, world, rank, gen, slot_floats, true,
                       fused_tail ? &e : nullptr);
    if (rc || fused_tail) return rc;
    return ep_combine_launch(rank, world, slots, flags, gen, f_own, R, layer->H, slot_floats, status, st, 1);
}

int hmoe_combine(float* f, const float* o, float* y, int64_t n, const float* o2, void* stream)
{
    if (!f || !y || n < 0 || n % 4) return fail(HMOE_E_ARG, "hmoe_combine: f, y and n % 4 == 0 required");
    if (n == 0) return HMOE_OK;
    {
        // behind the decode kernels (which release their dependents early) the launch latency overlaps the down kernel's tail
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned) ((n / 4 + 255) / 256)); cfg.blockDim = dim3(256); cfg.stream = (cudaStream_t) stream;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at; cfg.numAttrs = 1;
        cudaLaunchKernelEx(&cfg, combine_kernel, f, o, y, n, o2);
    }
    count_launches(1);
    const cudaError_t err = cudaGetLastError();
    return err == cudaSuccess ? HMOE_OK : fail(HMOE_E_CUDA, cudaGetErrorString(err));
}

int hmoe_combine_norm(const float* f, const float* o, float* y, const float* o2, float* r, const void* w, int w_dtype, void* xn, int rows, int H,
                      float eps, float cbias, float cscale, void* stream)
{
    if (!y || !r || !w || !xn || rows < 1 || H < 4 || H % 4 || H > 4 * NORM_THREADS * NORM_VECS)
        return fail(HMOE_E_ARG, "hmoe_combine_norm: y, r, w, xn required; H a multiple of 4, at most 16384");
    if (w_dtype != HMOE_F16 && w_dtype != HMOE_BF16) return fail(HMOE_E_ARG, "hmoe_combine_norm: the norm weight must be fp16 or bf16");
    NormParts in = {};
    in.part[0] = f; in.part[1] = y; in.n = 2;
    if (o) in.part[in.n++] = o;
    if (o2) in.part[in.n++] = o2;
    in.clear = y;
    if (w_dtype == HMOE_BF16) sum_norm_kernel<true><<<rows, NORM_THREADS, 0, (cudaStream_t) stream>>>(in, r, (const uint16_t*) w, (__half*) xn, H, eps, cbias, cscale);
    else sum_norm_kernel<false><<<rows, NORM_THREADS, 0, (cudaStream_t) stream>>>(in, r, (const uint16_t*) w, (__half*) xn, H, eps, cbias, cscale);
    count_launches(1);
    const cudaError_t err = cudaGetLastError();
    return err == cudaSuccess ? HMOE_OK : fail(HMOE_E_CUDA, cudaGetErrorString(err));
}

int hmoe_dequant(const void* q, const void* scales, int group, int scale_dtype, int N, int K, void* out_f16, void* stream)
{
    if (!q || !scales || !out_f16 || N % 64 || K % 64 || N <= 0 || K <= 0) return fail(HMOE_E_ARG, "hmoe_dequant: N and K must be multiples of 64");
    if (!(group == 0 && scale_dtype == HMOE_F32) && !(group > 0 && K % group == 0 && scale_dtype == HMOE_BF16))
        return fail(HMOE_E_ARG, "hmoe_dequant: scales must be fp32 per row (group 0) or bf16 per group");
    dequant_kernel<<<1024, 256, 0, (cudaStream_t) stream>>>((const uint4*) q, scales, group, N, K, (__half*) out_f16);
    count_launches(1);
    const cudaError_t err = cudaGetLastError();
    return err == cudaSuccess ? HMOE_OK : fail(HMOE_E_CUDA, cudaGetErrorString(err));
}

int hmoe_ws_status(void* ws, uint32_t* status_out, void* stream)
{
    if (!ws || !status_out) return fail(HMOE_E_ARG, "hmoe_ws_status: null pointer");
    uint32_t v = 0;
    cudaError_t err = cudaMemcpyAsync(&v, ws, 4, cudaMemcpyDeviceToHost, (cudaStream_t) stream);
    if (err == cudaSuccess) err = cudaMemsetAsync(ws, 0, 4, (cudaStream_t) stream);
    if (err == cudaSuccess) err = cudaStreamSynchronize((cudaStream_t) stream);
    if (err != cudaSuccess) return fail(HMOE_E_CUDA, cudaGetErrorString(err));
    *status_out = v;
    if (v & ST_WAIT_TIMEOUT) return fail(HMOE_E_TIMEOUT, "a bounded device-side wait gave up");
    return HMOE_OK;
}

int hmoe_fill_bytes(void* dst, size_t nbytes, uint64_t seed, uint64_t stream_id, void* stream)
{
    if (!dst || nbytes % 8) return fail(HMOE_E_ARG, "hmoe_fill_bytes: nbytes must be a multiple of 8");
    if (nbytes == 0) return HMOE_OK;
    // host-side copy of the generator's first step: base = mix(seed * G + stream_id)
    unsigned long long z = (unsigned long long) seed * 0x9E3779B97F4A7C15ull + (unsigned long long) stream_id;
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    fill_kernel<<<2048, 256, 0, (cudaStream_t) stream>>>((unsigned long long*) dst, nbytes / 8, z);
    count_launches(1);
    const cudaError_t err = cudaGetLastError();
    return err == cudaSuccess ? HMOE_OK : fail(HMOE_E_CUDA, cudaGetErrorString(err));
}

}  // extern "C"

#ifdef HMOE_PROBE_TIMELINE
using namespace hmoe;
TL_READER(hmoe_tl_combine)
#endif

/* hecate_moe.h - C ABI of libhecate_moe_b200.so: the MoE expert hot path of chronarion/hecate for NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain pointers and sizes, returns 0 (HMOE_OK) or an error code, never throws, never allocates
 * device memory and never synchronises the stream unless its comment says so. All device pointers must belong to the
 * current CUDA device. `stream` is a cudaStream_t passed as void*. hmoe_last_error() returns the message of the calling
 * thread's last failure. Paths in the comments name the reference interface each entry point replaces (relative to the
 * reference project's root).
 *
 * Weight format (unchanged from the reference): a matrix W[N][K] of 4-bit codes c (value c - 8) packed by
 * tools/quant/gptq_int4.py:74-77 (pack_u4); see hecate_b200/layout.py for the index formula. Scales are either one fp32
 * per row (group = 0, scale_dtype = HMOE_F32; the reference's format) or one bf16 per 128 input columns (group = 128,
 * scale_dtype = HMOE_BF16) stored [N/64][K/128][64]: the 64 scales of a 64-row group and one column group are contiguous,
 * row r of the group at position (r % 8) * 8 + r / 8, so that one 16-byte load gives a lane the eight rows it feeds to the
 * MMAs (hecate_b200/layout.py: group_scales_device_order). Every weight and scale pointer must be 16-byte aligned.
 */
#ifndef HECATE_MOE_H
#define HECATE_MOE_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { HMOE_OK = 0, HMOE_E_ARG = 1, HMOE_E_CUDA = 2, HMOE_E_TIMEOUT = 3, HMOE_E_WS = 4, HMOE_E_UNSUPPORTED = 5 };
enum { HMOE_F16 = 0, HMOE_BF16 = 1, HMOE_F32 = 2,
       HMOE_F16_FRAG = 3 /* hmoe_decode's x only: fp16 rows already in the MMA column order, as the reference's norm + router kernel
                            writes them for moe4.forward(xf = 1) (runtime/tier/moe4/moe4.cu:68-72, runtime/core/nr4_kernel.cuh:99-118) */ };

/* One MoE layer's experts as the reference's loader hands them to its kernels (runtime/tier/tier_split.py:206-246):
 * six device arrays of n_experts device pointers (int64), one per matrix and per scale tensor, plus the optional shared
 * expert (all six pointers null = none). gate/up are [I][H], down is [H][I]. */
typedef struct hmoe_layer
{
    int32_t H, I, n_experts, topk;
    int32_t group;        /* 0 = one scale per row, 128 = one scale per 128 input columns */
    int32_t scale_dtype;  /* HMOE_F32 with group 0, HMOE_BF16 with group 128 */
    const int64_t* gate_w; const int64_t* up_w; const int64_t* down_w;
    const int64_t* gate_s; const int64_t* up_s; const int64_t* down_s;
    const void* sh_gate_w; const void* sh_up_w; const void* sh_down_w;
    const void* sh_gate_s; const void* sh_up_s; const void* sh_down_s;
    int32_t shared_format; /* 0: the shared expert is stored like a routed expert (int4, the layer's scale format);
                              1: the reference's own shared expert (runtime/tier/tier_split.py:495-514): int8 codes (value = code - 128)
                              in its dense GEMV fragment order with one fp32 scale per output row (decode and prefill) */
} hmoe_layer;

int hmoe_version(void);
const char* hmoe_last_error(void);
/* Kernels launched by this library in this process so far (for benchmark bookkeeping). */
int64_t hmoe_launch_count(void);

/* Router: replaces router_fused(x, wt, bias, logits, ctr, sel, rw, topk, scale) (runtime/core/exl3_router.py:134-146) and the
 * routing_dots contract (docker/patches/exllamav3/block_sparse_mlp_routing.py:253-301) for any number of rows.
 * x [R][H] and wt [E][H] are fp16 or bf16 (x_dtype / w_dtype), bias fp32 [E] or null. Writes sel int64 [R][topk] (selection
 * order: descending sigmoid(logit) + bias, ties to the lower expert id) and rw fp16 [R][topk] = act * scale / (sum + 1e-20).
 * Needs E % 32 == 0, E <= 256, H % 256 == 0, topk <= 8. ws: hmoe_router_ws_bytes(R, E) bytes of device scratch, zero-filled once
 * before first use; its first word is a status word (hmoe_ws_status): if a bounded wait inside the kernel gives up, bit 0 is
 * set and the call writes no selection. */
size_t hmoe_router_ws_bytes(int R, int E);
int hmoe_router(const void* x, int x_dtype, const void* wt, int w_dtype, const float* bias, int R, int H, int E, int topk,
                float scale, int64_t* sel, void* rw, void* ws, size_t ws_bytes, void* stream);

/* Residual add + input norm + router in one launch: the step the reference fuses as norm_route (runtime/core/exl3_normroute.py:16-65,
 * runtime/core/nr4_kernel.cuh:121-381). r' = r + y (y may be null), xn = fp16(r' * (nw + cbias) * rsqrt(mean(r'^2) + eps) * cscale),
 * then hmoe_router on xn. r, y fp32 [R][H] are only read; r' goes to r_out (fp32 [R][H], may be null, must not alias r or y), xn
 * fp16 [R][H] is the expert layer's input. The sum of squares is taken in the order of hmoe_combine_norm and the router sees the
 * fp16-rounded xn, so the results equal those of the two separate calls bit for bit. H <= 6144; other limits as hmoe_router. */
int hmoe_norm_router(const float* y, const float* r, float* r_out, const void* nw, int nw_dtype, void* xn, const void* wt, int w_dtype,
                     const float* bias, int R, int H, int E, int topk, float scale, float eps, float cbias, float cscale, int64_t* sel, void* rw,
                     void* ws, size_t ws_bytes, void* stream);

/* Decode expert layer: replaces moe4.forward(x, sel, rw, n_hot, tables..., scratch..., y, blocks, blocks_a, lo, shared...)
 * (runtime/tier/moe4/moe4.cu:828-895) for R <= 16 rows in one pass over the weights. x [R][H] fp16 or bf16 (or HMOE_F16_FRAG); sel int64
 * [R][topk]; rw fp16 [R][topk]; only ids in [lo, lo + n_local) contribute, entry e - lo of the tables; y fp32 [R][H] is
 * accumulated into. act_quant = 1 reproduces the reference CPU engine's int8 activation round trips
 * (runtime/tier/cpuband.cpp:106-111,140-150,200-207); 0 keeps fp16 activations like the reference GPU kernels.
 * ws: hmoe_decode_ws_bytes(H, I) bytes, zero-filled once before first use (replaces moe4.scratch, moe4.cu:897-902). */
size_t hmoe_decode_ws_bytes(int H, int I);
int hmoe_decode(const hmoe_layer* layer, const void* x, int x_dtype, const int64_t* sel, const void* rw, int R, int lo, int n_local,
                int act_quant, float* y, void* ws, size_t ws_bytes, void* stream);

/* hmoe_router followed by hmoe_decode on the router's own output, as three launches instead of four: the router's launch also
 * does the decode call's set-up step (the rows rewritten for the MMAs by one more block per row group while the logits are
 * computed; the work list built by the block that completes the last selection), so no separate set-up kernel sits between
 * the router and the expert kernels. This is what the reference's hooks do back to back per layer: routing_fn, then
 * cpu_split_submit with the selection it returned (docker/patches/exllamav3/block_sparse_mlp_routing.py:253-301,
 * runtime/tier/tier_split.py:520-574). Arguments as in the two calls; H and topk are the layer's; R <= 16; sel and rw are outputs.
 * A wait that gives up inside the router sets bit 0 of the decode workspace's status word and the call computes nothing. */
int hmoe_router_decode(const hmoe_layer* layer, const void* x, int x_dtype, const void* wt, int w_dtype, const float* bias, int R, int E, float scale,
                       int64_t* sel, void* rw, void* router_ws, size_t router_ws_bytes, int lo, int n_local, int act_quant, float* y, void* ws,
                       size_t ws_bytes, void* stream);

/* Expert-parallel decode over the GPUs of one box (no reference counterpart as such: the reference splits a layer's experts
 * over unlike processors that all receive every row and ignore foreign ids, runtime/tier/tier_split.py:3-11, moe4.cu:93, and
 * adds their fp32 partials in a fixed order, moe4.cu:702-717; these entry points do the same over NVLink peer memory).
 * hmoe_decode_ep = hmoe_decode where the shared expert only takes rows r with r % shared_mod == shared_rem (each rank serves
 * its share of the rows; experts are split by lo / n_local), y is the base of this rank's two partial slots (slot_floats
 * apart) and gen a device word: the call adds 1 to *gen and writes its partial into slot *gen % 2. hmoe_ep_alloc / export /
 * open / close manage the symmetric buffers (cudaMalloc + CUDA IPC; set-up time only). hmoe_ep_combine(rank, world, slots,
 * flags, gen, f, rows, H, slot_floats, status, stream): slots[p] / flags[p] are rank p's buffers as seen from this process (own
 * pointers for p == rank): two zero-initialised fp32 slots and `world` uint32 flags. It reads the generation g from *gen,
 * publishes it to every peer, waits at most 2 s until all peers have published g, adds all ranks' partials of slot g % 2 to f
 * in rank order and clears the other slot. All ranks must make the same sequence of steps. A wait that gives up sets bit 0 of
 * *status (device word). Neither call keeps host-side state, so a step can be captured in a CUDA graph. */
int hmoe_decode_ep(const hmoe_layer* layer, const void* x, int x_dtype, const int64_t* sel, const void* rw, int R, int lo, int n_local,
                   int act_quant, float* y, void* ws, size_t ws_bytes, int shared_mod, int shared_rem, uint32_t* gen, size_t slot_floats,
                   void* stream);
int hmoe_ep_alloc(size_t bytes, void** ptr);
int hmoe_ep_free(void* ptr);
int hmoe_ep_export(void* ptr, unsigned char* handle64);
int hmoe_ep_open(const unsigned char* handle64, void** ptr);
int hmoe_ep_close(void* ptr);
int hmoe_ep_combine(int rank, int world, void* const* slots, void* const* flags, const uint32_t* gen, float* f, int rows, int H, size_t slot_floats,
                    uint32_t* status, void* stream);

/* The token exchange of expert-parallel decode as an all-to-all over NVLink peer memory (no reference counterpart as such; the
 * shape kept is the reference's mailbox: a per-layer slot with the rows, their selections and weights, and an ISSUE flag stored
 * with release semantics at system scope, runtime/tier/moe4/moe4.cu:719-738, runtime/tier/rtx_graph.py:105-134). Tokens are
 * data-parallel: of a step's R <= 16 rows, rank r holds rows r, r + world, ... (x_own [n][H] 2-byte elements, sel_own int64
 * [n][topk], rw_own fp16 [n][topk], compact, produced by the rank's own router call).
 * hmoe_ep_dispatch: stores the rank's rows into every rank's staging area (stage[p] = rank p's area as seen from this process,
 * hmoe_ep_stage_bytes(H, topk) bytes from hmoe_ep_alloc, zero at start), raises its flag there and waits, at most 2 s (then bit 0
 * of *status), until every rank's rows have arrived here. Afterwards the local area holds x [R][H], sel [R][topk], rw [R][topk] at
 * the offsets hmoe_ep_stage_offsets returns: the inputs of hmoe_decode_ep. All ranks must make the same sequence of steps, each
 * followed by a combine (which is what makes a single staging area enough).
 * hmoe_ep_combine_own: hmoe_ep_combine for data-parallel tokens: f_own [n][H] += the sums of this rank's rows only. */
/* hmoe_decode_ep followed by hmoe_ep_combine (own_rows = 0) or hmoe_ep_combine_own (own_rows = 1) as one call without the
 * combine's launch: the down kernel's blocks do the combine when they run out of weights to stream (the block that finishes last
 * raises the flags, every block waits, bounded, for the peers and sums its slice of the peers' partials into f). Same buffers and
 * protocol as the separate calls, so ranks using either form interoperate step by step. Needs H <= 6144 and I <= 2048. */
int hmoe_decode_ep_combine(const hmoe_layer* layer, const void* x, int x_dtype, const int64_t* sel, const void* rw, int R, int lo, int n_local,
                           int act_quant, void* ws, size_t ws_bytes, int shared_mod, int shared_rem, uint32_t* gen, size_t slot_floats, int rank,
                           int world, void* const* slots, void* const* flags, float* f, int own_rows, uint32_t* status, void* stream);
/* One expert-parallel decode layer call with data-parallel tokens, end to end, in four launches: dispatch + router + set-up (one
 * kernel: blocks (p, 0) store this rank's rows x_own [n][H] into rank p's staging area and raise the flag there; every block waits,
 * bounded, for the owners of the rows it needs; every rank then routes all R rows, which costs what routing its own would, and
 * builds its work list), gate_up, down, and the combine of the rank's own rows (fused_tail != 0: inside the down launch).
 * sel int64 [R][topk] and rw fp16 [R][topk] receive the routing of all rows; f_own [n][H] += the layer output of this rank's rows
 * (rows rank, rank + world, ...). Buffers as in hmoe_ep_dispatch / hmoe_decode_ep / hmoe_ep_combine_own, with which it can be mixed
 * step by step. A wait that gives up sets bit 0 of the decode workspace's status word or of *status.
 * Two holders per expert: with n_local == 2 * E / world (and lo == rank * E / world, E <= 256) the rank's tables hold the bands
 * rank and rank + 1 (mod world) of E / world router positions each, in this order, so every expert is held by two ranks; each step
 * every rank derives from the (identical) selections which holder serves each picked expert: the bands walk their positions side by
 * side and give each picked one to the holder with fewer experts so far. Twice the weight memory, most loaded rank 26.1 instead of
 * 29.5 experts at 4 ranks and 13.8 instead of 16.7 at 8 (16 rows, random top-8). */
int hmoe_decode_ep_dp(const hmoe_layer* layer, const void* x_own, int x_dtype, const void* wt, int w_dtype, const float* bias, int R, int E,
                      float scale, int64_t* sel, void* rw, void* router_ws, size_t router_ws_bytes, int lo, int n_local, int act_quant, void* ws,
                      size_t ws_bytes, int rank, int world, void* const* stage, void* const* slots, void* const* flags, uint32_t* gen,
                      size_t slot_floats, float* f_own, uint32_t* status, int fused_tail, void* stream);
size_t hmoe_ep_stage_bytes(int H, int topk);
int hmoe_ep_stage_offsets(int H, int topk, size_t* x_off, size_t* sel_off, size_t* rw_off);
int hmoe_ep_dispatch(int rank, int world, void* const* stage, const void* x_own, const int64_t* sel_own, const void* rw_own, int R, int H, int topk,
                     uint32_t* status, void* stream);
int hmoe_ep_combine_own(int rank, int world, void* const* slots, void* const* flags, const uint32_t* gen, float* f_own, int rows, int H,
                        size_t slot_floats, uint32_t* status, void* stream);

/* Prefill permutation on the device: replaces the host-side code of runtime/tier/tier_split.py:404-412,433-455 (stable argsort
 * of the flattened selection by expert id, bincount with a host sync) and pick_groups (runtime/tier/rtx_split.py:236-255, one
 * pick group) with three kernels and no synchronisation. Picks with ids outside [lo, lo + n_local) are dropped.
 * Outputs (device, caller-owned): order int32 [R*topk] (flat pick index, may be null), tok int32 [R*topk + shared_rows]
 * (= order / topk), eid int32 (local expert id; n_local for the shared expert's rows), wt fp32, counts int32 [n_local + 1],
 * rbt int32 [maxrb][4] = {expert, first pick, picks <= bm, 0} with maxrb >= (R*topk + shared_rows) / bm + n_local + 2,
 * plan int32 [4] = {picks kept + shared rows, row blocks, 0, 0}. shared_rows > 0 appends a segment "every row once, weight 1"
 * as expert n_local. balance != 0: an expert's blocks get near-equal sizes. ws: hmoe_permute_ws_bytes bytes. */
size_t hmoe_permute_ws_bytes(int R, int topk, int n_local);
int hmoe_permute(const int64_t* sel, const void* rw, int R, int topk, int lo, int n_local, int shared_rows, int bm, int balance,
                 int32_t* order, int32_t* tok, int32_t* eid, float* wt, int32_t* counts, int32_t* rbt, int32_t* plan, void* ws, size_t ws_bytes,
                 void* stream);

/* Prefill expert layer: replaces moe4t.forward / moe4p.forward(x, tok, eid, wt, rbt, gw, uw, dw, gs, us, ds, gu, ar, d, out)
 * (runtime/tier/moe4/moe4t.cu:498-524, moe4p.cu:220-245) together with the permutation above, for any number of rows:
 * permute -> gather -> grouped gate+up GEMM with SiLU * up * weight epilogue -> grouped down GEMM whose epilogue adds
 * scale * sum into out[token] (fp32 [R][H], added into: zero it first for a plain result). tcgen05 tensor cores, fp16
 * operands, fp32 accumulation. act_quant = 1 reproduces the CPU engine's int8 activation round trips: code x scale is carried
 * as an fp16 hi + lo pair and the weights are walked twice (twice the tensor-core work; a parity mode, not the fast path).
 * Other arguments as hmoe_decode. ws: hmoe_prefill_ws_bytes(..., act_quant) bytes (holds the gathered inputs and the
 * intermediate activations: (R*topk + R) * (H + I) * 2 bytes, twice that in the int8 mode, plus small tables). */
size_t hmoe_prefill_ws_bytes(int R, int topk, int n_local, int H, int I, int act_quant);
int hmoe_prefill(const hmoe_layer* layer, const void* x, int x_dtype, const int64_t* sel, const void* rw, int R, int lo, int n_local,
                 int act_quant, float* out, void* ws, size_t ws_bytes, void* stream);

/* Short prefill: the range between a decode call and the grouped GEMMs, 1..640 rows (replaces the branch of _hot_prefill,
 * runtime/tier/tier_split.py:341-355, that runs 9..64 rows through moe4.forward in 8-row chunks, each chunk streaming its
 * experts again). The whole call is one list of (expert, <= 8 picks) tiles for the decode streaming kernels, so a distinct
 * expert is read from memory once per eight of its picks; the grouped GEMMs convert every expert's weights whatever its row
 * count and only win from several hundred rows up (level at about 640 rows of uniform routing over 256 experts). Arguments as hmoe_prefill (out is added into). Needs H <= 6144, I <= 2048
 * (else HMOE_E_UNSUPPORTED); the int8 shared expert runs sixteen rows at a time through the decode path's kernels and is not
 * available with act_quant = 1 (nor in hmoe_decode; hmoe_prefill and hmoe_forward serve that combination). ws: hmoe_short_prefill_ws_bytes(R, ...) bytes, 0 for R outside 1..640. */
size_t hmoe_short_prefill_ws_bytes(int R, int H, int I, int topk);
int hmoe_short_prefill(const hmoe_layer* layer, const void* x, int x_dtype, const int64_t* sel, const void* rw, int R, int lo, int n_local,
                       int act_quant, float* out, void* ws, size_t ws_bytes, void* stream);

/* hmoe_short_prefill for one rank of an expert-parallel group (no reference counterpart), as hmoe_prefill_ep: experts split by
 * lo / n_local, the shared expert applied to rows [shared_row0, shared_row0 + shared_rows) only (the rank's own tokens). */
int hmoe_short_prefill_ep(const hmoe_layer* layer, const void* x, int x_dtype, const int64_t* sel, const void* rw, int R, int lo, int n_local,
                          int act_quant, float* out, void* ws, size_t ws_bytes, int shared_row0, int shared_rows, void* stream);

/* One entry point for any number of rows, as tier_submit / _hot_prefill choose among the reference's kernels by row count
 * (runtime/tier/tier_split.py:341-364,543-546): R <= 16 -> hmoe_decode, R <= hmoe_forward_short_rows() -> hmoe_short_prefill
 * (256 with the int8 shared expert; when the layer's shapes allow it), else hmoe_prefill; the int8 shared expert with act_quant = 1 always takes hmoe_prefill. One workspace serves every row count up to
 * the R it was sized for: hmoe_forward_ws_bytes(R_max, ...) bytes, zero-filled once. */
int hmoe_forward_short_rows(void);
size_t hmoe_forward_ws_bytes(int R, int topk, int n_local, int H, int I, int act_quant);
int hmoe_forward(const hmoe_layer* layer, const void* x, int x_dtype, const int64_t* sel, const void* rw, int R, int lo, int n_local,
                 int act_quant, float* out, void* ws, size_t ws_bytes, void* stream);

/* hmoe_prefill for one rank of an expert-parallel group (no reference counterpart): experts split by lo / n_local as above;
 * the shared expert is applied to rows [shared_row0, shared_row0 + shared_rows) only (the rank's own tokens). */
int hmoe_prefill_ep(const hmoe_layer* layer, const void* x, int x_dtype, const int64_t* sel, const void* rw, int R, int lo, int n_local,
                    int act_quant, float* out, void* ws, size_t ws_bytes, int shared_row0, int shared_rows, void* stream);

/* hmoe_prefill_ep with the combine fused into the down GEMM (no reference counterpart): row t of the R = world * rows_per_rank
 * gathered rows belongs to rank t / rows_per_rank, and its sums are added straight into that rank's output
 * out_peer[rank][t % rows_per_rank][H] with fp32 reductions over NVLink peer memory (out_peer: host array of `world` device
 * pointers, the own one and the peers' opened with hmoe_ep_open). Every rank zeroes its own output before the step's first
 * collective and calls hmoe_ep_barrier after this call; its output is complete when the barrier has passed.
 * hmoe_ep_barrier: raises generation `gen` (a number that grows by one per step) in every peer's flag array (flags[p] =
 * rank p's array of `world` words, zero at start) and waits, at most 2 s, until every peer has raised it here; on a
 * time-out bit 0 of *status is set and the kernel returns. */
int hmoe_prefill_ep_peer(const hmoe_layer* layer, const void* x, int x_dtype, const int64_t* sel, const void* rw, int R, int lo, int n_local,
                         int act_quant, void* const* out_peer, int world, int rows_per_rank, void* ws, size_t ws_bytes, int shared_row0,
                         int shared_rows, void* stream);
int hmoe_ep_barrier(int rank, int world, void* const* flags, uint32_t gen, uint32_t* status, void* stream);
/* Prefill dispatch as an all-to-all-v over NVLink peer memory (no reference counterpart; the mailbox of runtime/tier/moe4/moe4.cu:719-738
 * is its template: payload stored into the consumer's memory, then a flag). Every rank holds rows_per_rank rows (rank r the global
 * rows [r * rows_per_rank, (r + 1) * rows_per_rank)) and stores each of them, at its global position, into the staging area of every
 * rank that holds one of the row's selected experts (router position e belongs to rank e / n_per_rank; ids outside
 * [0, world * n_per_rank) select no rank) and into its own; selections and weights go to every rank. stage[p] = rank p's staging area
 * as seen from this process (hmoe_prefill_ep_stage_bytes from hmoe_ep_alloc): x [R][H] 16-bit at offset 0, sel int64 [R][topk] and
 * rw 16-bit [R][topk] at the offsets hmoe_prefill_ep_stage_offsets returns; these are then the x / sel / rw of hmoe_prefill_ep(_peer)
 * with R = world * rows_per_rank. A rank never reads rows it was not sent: its permutation lists only rows with a local expert, and
 * the shared expert is applied to the rank's own rows. Call hmoe_ep_barrier after it (it publishes the stores); the next step's
 * dispatch may start once every rank has finished reading its staging area (e.g. after the barrier that ends the peer combine, or
 * after the reduce-scatter). sent_rows (device counter, may be null) is increased by the number of (row, remote rank) pairs stored. */
size_t hmoe_prefill_ep_stage_bytes(int rows_total, int H, int topk);
int hmoe_prefill_ep_stage_offsets(int rows_total, int H, int topk, size_t* sel_off, size_t* rw_off);
int hmoe_prefill_ep_dispatch(int rank, int world, void* const* stage, const void* x_own, const int64_t* sel_own, const void* rw_own, int rows_per_rank,
                             int H, int topk, int n_per_rank, unsigned long long* sent_rows, void* stream);
/* Stream-ordered memset / device-to-device copy for memory obtained from hmoe_ep_alloc (which the host language may have no
 * tensor for). */
int hmoe_ep_memset(void* ptr, int value, size_t bytes, void* stream);
int hmoe_ep_copy(void* dst, const void* src, size_t bytes, void* stream);

/* The same two grouped GEMMs with the reference's calling convention, for callers that keep the reference's host-side
 * permutation: replaces moe4t.forward / moe4p.forward(x, tok, eid, wt, rbt, gw, uw, dw, gs, us, ds, gu, ar, d, out)
 * (runtime/tier/moe4/moe4t.cu:498-524). tok int32 [npos] (token of each sorted pick), wt fp32 [npos], rbt int32 [nrb][4] =
 * {expert, first pick, picks <= 256, 0}, all on the device; the expert of a pick is taken from its row block (eid is not
 * needed). Expert ids >= n_local select the shared expert. ws: hmoe_prefill_sorted_ws_bytes(npos, H, I) (replaces
 * moe4t.scratch, moe4t.cu:490-495). */
size_t hmoe_prefill_sorted_ws_bytes(int npos, int H, int I, int act_quant);
int hmoe_prefill_sorted(const hmoe_layer* layer, const void* x, int x_dtype, const int32_t* tok, const float* wt, const int32_t* rbt, int nrb,
                        int npos, int n_local, int act_quant, float* out, void* ws, size_t ws_bytes, void* stream);

/* hmoe_decode without a workspace argument, for callers that cannot allocate device memory: embedders whose device memory
 * is one arena planned at start-up, plugins that must stay inside a host framework's allocator, latency-critical loops
 * where an allocation would stall the process. It has no counterpart in the reference (whose scratch always comes from
 * torch, runtime/tier/moe4/moe4.cu:897-902). The workspace is a 5 MiB array built into the library image (held by every GPU
 * that loads the library), which limits it to decode_ws_bytes(H, I) <= 5 MiB, i.e. up to H = 6144 with I = 2048; larger
 * shapes are refused with HMOE_E_WS. Same arguments and results as hmoe_decode otherwise. status_dev, if not null, is a
 * caller-owned 4-byte device word that receives the call's status bits (see hmoe_ws_status) on the same stream.
 * The first call on each device looks up the array's device address (a one-time set-up; make that call outside stream
 * capture). It allocates nothing, ever. All calls on a device share the array: calls that overlap on the GPU race. */
int hmoe_decode_noalloc(const hmoe_layer* layer, const void* x, int x_dtype, const int64_t* sel, const void* rw, int R, int lo,
                        int n_local, int act_quant, float* y, uint32_t* status_dev, void* stream);

/* Phase timing of the decode path (no reference counterpart; the reference uses compile-time ablation macros,
 * runtime/tier/moe4/moe4.cu:6-10). With profiling on, each hmoe_decode call records CUDA events between its three kernels
 * on the caller's stream, into a ring of 32 sets; hmoe_decode_phase_times waits for them and returns the durations in ms
 * of {prepare, gate_up, down} averaged over the calls made since profiling was switched on (at most the last 32). While
 * profiling is on the kernels are launched without programmatic overlap, so each duration is that of the kernel alone.
 * The first switch-on creates the events (allocates; call it outside stream capture). */
int hmoe_set_profiling(int on);
int hmoe_decode_phase_times(float* ms3);

/* Combine: replaces moe4.combine(f, o_ptr, y, rows, o2_ptr, done_ptr) (runtime/tier/moe4/moe4.cu:702-717,817-824):
 * f += y (+ o) (+ o2) in that order, then y = 0. o and o2 may be null. n = rows * H must be a multiple of 4. */
int hmoe_combine(float* f, const float* o, float* y, int64_t n, const float* o2, void* stream);

/* The combine fused into the next layer's input norm: replaces combine_norm(f, o_ptr, y, rows, o2_ptr, done_ptr, r, w, xn, eps,
 * cbias, cscale) (runtime/tier/cn.cu:50-105,190-210). Per row: a = ((f + y) + o) + o2 (f, o, o2 may be null), y = 0,
 * r += a (fp32 residual [rows][H], in place), xn = fp16(r * (w + cbias) * rsqrt(mean(r^2) + eps) * cscale), w fp16 or bf16 [H].
 * Same column ownership and summation order as the reference kernel. H % 4 == 0, H <= 16384. f is not written. */
int hmoe_combine_norm(const float* f, const float* o, float* y, const float* o2, float* r, const void* w, int w_dtype, void* xn, int rows, int H,
                      float eps, float cbias, float cscale, void* stream);

/* Dequantise one packed matrix to fp16 [N][K] (value * scale): replaces moe4.dequant(q, sc, N, K)
 * (runtime/tier/moe4/moe4.cu:679-698,904-911); group / scale_dtype as in hmoe_layer. */
int hmoe_dequant(const void* q, const void* scales, int group, int scale_dtype, int N, int K, void* out_f16, void* stream);

/* Reads and clears the status word kernels set when a bounded device-side wait gave up or an index was out of range
 * (synchronises the stream). *status_out: bit 0 = wait timed out, bit 1 = bad index. Returns HMOE_E_TIMEOUT if bit 0 is set. */
int hmoe_ws_status(void* ws, uint32_t* status_out, void* stream);

/* Synthetic data: fills nbytes (multiple of 8) with the counter-based generator of hecate_b200/synth.py
 * (word i = mix(mix(seed * G + stream_id) + i)), identical to the numpy implementation. No reference counterpart. */
int hmoe_fill_bytes(void* dst, size_t nbytes, uint64_t seed, uint64_t stream_id, void* stream);

#ifdef __cplusplus
}
#endif
#endif

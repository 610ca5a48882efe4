// Internal host-side declarations shared by the translation units of libhecate_moe_b200.so.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>
#include "../../include/hecate_moe.h"

namespace hmoe {

// records the message for hmoe_last_error() and returns `code`
int fail(int code, const char* msg);
void count_launches(int n);

// Per-device host state. One process may drive several GPUs through this library, so nothing that belongs to a device (its SM
// count, whether a kernel's shared-memory attribute has been set there) is kept in a per-process static.
constexpr int MAX_DEVICES = 64;
int current_device();                     // cudaGetDevice, -1 on failure
int device_sms();                         // SM count of the current device (looked up once per device)
// One flag per device: first() is true the first time it is called with a given device current (and every time for device
// numbers beyond MAX_DEVICES, where the set-up it guards is simply repeated).
struct DeviceOnce
{
    unsigned char done[MAX_DEVICES] = {};
    bool first()
    {
        const int d = current_device();
        if (d < 0 || d >= MAX_DEVICES) return true;
        if (done[d]) return false;
        done[d] = 1;
        return true;
    }
};

// the expert-parallel combine as the tail of the down launch (hmoe_decode_ep_combine)
struct EpCombineArgs
{
    int rank, world, own_rows;
    void* const* slots; void* const* flags;
    float* f;
    unsigned* status;
};

size_t decode_ws_bytes(int H, int I);
size_t short_ws_bytes(int R, int H, int I, int topk);
int short_launch(const hmoe_layer* L, const void* x, int x_dtype, const int64_t* sel, const void* rw, int R, int lo, int n_local,
                 int act_quant, float* y, void* ws, size_t ws_bytes, cudaStream_t st, int shared_row0 = 0, int shared_rows = -1);
int decode_launch(const hmoe_layer* L, const void* x, int x_dtype, const int64_t* sel, const void* rw, int R, int lo, int n_local,
                  int act_quant, float* y, void* ws, size_t ws_bytes, cudaStream_t st, int sh_mod = 1, int sh_rem = 0,
                  unsigned* gen_ptr = nullptr, size_t slot_stride = 0, bool prepared = false, const struct EpCombineArgs* epc = nullptr);
struct PrepArgs;
struct DispArgs;
int decode_prep_args(const hmoe_layer* L, const void* x, int x_dtype, int R, int lo, int n_local, int act_quant, void* ws, size_t ws_bytes,
                     int sh_mod, int sh_rem, unsigned* gen_ptr, PrepArgs* pa);
int router_prepare_launch(const void* x, int x_dtype, const void* wt, int w_dtype, const float* bias, int R, int H, int E, int topk, float scale,
                          int64_t* sel, void* rw, void* ws, size_t ws_bytes, const PrepArgs& pa, cudaStream_t st, const DispArgs* da = nullptr);
int ep_combine_launch(int rank, int world, void* const* slots, void* const* flags, const unsigned* gen, float* f, int rows, int H, size_t slot_floats,
                      unsigned* status, cudaStream_t st, int own_rows);

int shared_i8_launch(const hmoe_layer* L, int R, int sh_mod, int sh_rem, const __half* xf, float* gs, float* y, const unsigned* gen_ptr,
                     size_t slot_stride, int sms, cudaStream_t st);

int decode_set_profiling(int on);
int decode_phase_times(float* ms3);

size_t router_ws_bytes(int R, int E);
int router_launch(const void* x, int x_dtype, const void* wt, int w_dtype, const float* bias, int R, int H, int E, int topk,
                  float scale, int64_t* sel, void* rw, void* ws, size_t ws_bytes, cudaStream_t st);

int norm_router_launch(const float* y, const float* r, float* r_out, const void* nw, int nw_dtype, void* xn, const void* wt, int w_dtype,
                       const float* bias, int R, int H, int E, int topk, float scale, float eps, float cbias, float cscale, int64_t* sel, void* rw,
                       void* ws, size_t ws_bytes, cudaStream_t st);

size_t prefill_ws_bytes(int R, int topk, int n_local, int H, int I, int act_quant);
int prefill_launch(const hmoe_layer* L, const void* x, int x_dtype, const int64_t* sel, const void* rw, int R, int lo, int n_local,
                   int act_quant, float* out, void* ws, size_t ws_bytes, cudaStream_t st, int shared_row0 = 0, int shared_rows = -1,
                   void* const* out_peer = nullptr, int world = 1, int rows_per_rank = 0);
int ep_barrier_launch(int rank, int world, void* const* flags, unsigned gen, unsigned* status, cudaStream_t st);
size_t prefill_sorted_ws_bytes(int npos, int H, int I, int act_quant);
int prefill_sorted_launch(const hmoe_layer* L, const void* x, int x_dtype, const int32_t* tok, const float* wt, const int32_t* rbt, int nrb,
                          int npos, int n_local, int act_quant, float* out, void* ws, size_t ws_bytes, cudaStream_t st);
size_t permute_ws_bytes(int R, int topk, int n_local);
int permute_launch(const int64_t* sel, const void* rw, int R, int topk, int lo, int n_local, int shared_rows, int bm, int balance,
                   int32_t* order, int32_t* tok, int32_t* eid, float* wt, int32_t* counts, int32_t* rbt, int32_t* plan2, void* ws, size_t ws_bytes,
                   cudaStream_t st);

}  // namespace hmoe

// TEST INFRASTRUCTURE, NOT PRODUCT CODE.
// CPU restatement of the reference's MoE expert path, used only as the checker in tests, in the smoke test and as the
// timed CPU baseline. Nothing in the shipped library links or calls it.
//
// What it restates (paths are relative to the reference project):
//   * the Grace-CPU expert engine, runtime/tier/cpuband.cpp:80-111 (gemv_rows, quant_group), :153-177 (pick order,
//     summing the weights of repeated picks), :188-218 (the four phases and the pick-order accumulation);
//   * the packed int4 layout, tools/quant/gptq_int4.py:74-77 (pack_u4) and runtime/tier/tier_split.py:98-106
//     (_unpack_moe4 / _rowmajor_i4);
//   * the router contract of runtime/core/exl3_router.py:21-131 (sigmoid + bias keys, key-descending / index-ascending
//     top-k, renormalised fp16 weights) with a fixed summation order that the CUDA router follows exactly;
//   * the prefill permutation of runtime/tier/tier_split.py:404-412 and the row-block builder
//     runtime/tier/rtx_split.py:236-255 (pick_groups).
// Parity pin: orc_moe_job in q8 mode is bit-identical to the reference engine compiled from its own source (the
// oracle/_ref build) on every seeded case of tests/golden, and the permutation / layout functions reproduce vectors
// produced by executing the reference's own Python functions.
//
// Extensions beyond the reference, needed by the benchmark format: scales per group of G input columns (logical
// [K/G][N]; G = 0 means one scale per row, the reference's format, reproduced bit for bit), any number of rows (processed as
// independent jobs of <= 8 rows like the reference does), generic H / I, an exact mode (no activation quantisation,
// double accumulation) and an optional shared expert.
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

inline float h2f(uint16_t h) { _Float16 v; memcpy(&v, &h, 2); return (float) v; }
inline uint16_t f2h(float f) { _Float16 v = (_Float16) f; uint16_t h; memcpy(&h, &v, 2); return h; }

// cpuband.cpp:106-111
inline void quant_group32(const float* v, int8_t* q, float* sc)
{
    float m = 0.f;
    for (int k = 0; k < 32; ++k) m = fmaxf(m, fabsf(v[k]));
    const float s = m > 0 ? m / 127.f : 1.f;
    *sc = s;
    const float inv = 1.f / s;
    for (int k = 0; k < 32; ++k) q[k] = (int8_t) lrintf(v[k] * inv);
}

// One output row of cpuband.cpp:80-104 for one activation row, with a scale per group of G columns.
// The reference keeps four fp32 lanes: lane i of a 32-column group gathers columns 4i..4i+3 and 16+4i..16+4i+3 as an
// exact int32 dot product, which is then multiplied by the activation group scale with one fused multiply-add per lane;
// the row result is s[n] * ((l0 + l1) + (l2 + l3)). Here the four lanes restart at every weight-scale group and the group
// results are added in order, which is the same arithmetic when G == K.
inline float row_dot_q8(const uint8_t* qr, const float* srow, size_t sstride, int K, int G, const int8_t* xq, const float* xg)
{
    float tot = 0.f;
    for (int k0 = 0; k0 < K; k0 += G)
    {
        float lane[4] = {0.f, 0.f, 0.f, 0.f};
        for (int k = k0; k < k0 + G; k += 32)
        {
            int32_t d[4] = {0, 0, 0, 0};
            for (int j = 0; j < 32; ++j)
            {
                const uint8_t b = qr[(k + j) >> 1];
                const int c = (int) ((j & 1) ? (b >> 4) : (b & 15)) - 8;
                d[(j & 15) >> 2] += c * (int) xq[k + j];
            }
            const float g = xg[k / 32];
            for (int i = 0; i < 4; ++i) lane[i] = fmaf((float) d[i], g, lane[i]);
        }
        const float v = srow[(size_t) (k0 / G) * sstride] * ((lane[0] + lane[1]) + (lane[2] + lane[3]));
        tot = (k0 == 0) ? v : tot + v;
    }
    return tot;
}

inline double row_dot_exact(const uint8_t* qr, const float* srow, size_t sstride, int K, int G, const double* x)
{
    double tot = 0.0;
    for (int k0 = 0; k0 < K; k0 += G)
    {
        double a = 0.0;
        for (int k = k0; k < k0 + G; ++k)
        {
            const uint8_t b = qr[k >> 1];
            const int c = (int) ((k & 1) ? (b >> 4) : (b & 15)) - 8;
            a += (double) c * x[k];
        }
        tot += (double) srow[(size_t) (k0 / G) * sstride] * a;
    }
    return tot;
}

}  // namespace

extern "C" {

// One expert: row-major int4 codes (two per byte, low nibble = even column; tier_split.py:103-106) and fp32 scales laid
// out [K/G][N] (column-group major).
struct orc_expert
{
    const uint8_t* g; const uint8_t* u; const uint8_t* d;
    const float* gs; const float* us; const float* ds;
};

// Fragment-order packed codes -> row-major codes (inverse of pack_u4; tier_split.py:98-106). q holds N*K/2 bytes.
// Byte b = ((((((gr*KB + kb)*4 + s)*8 + g)*4 + q)*4 + t)*2 + cc)*2 + h, nibble rh, holds row gr*64 + s*16 + rh*8 + g and
// column kb*64 + t*16 + h*8 + q*2 + cc.
void orc_unpack_u4(const uint8_t* q, int N, int K, uint8_t* rowmajor)
{
    const int KB = K / 64;
    memset(rowmajor, 0, (size_t) N * K / 2);
    for (int n = 0; n < N; ++n)
        for (int k = 0; k < K; ++k)
        {
            const int gr = n / 64, s = (n % 64) / 16, rh = (n % 16) / 8, g = n % 8;
            const int kb = k / 64, t = (k % 64) / 16, h = (k % 16) / 8, qq = (k % 8) / 2, cc = k % 2;
            const size_t b = ((((((size_t) (gr * KB + kb) * 4 + s) * 8 + g) * 4 + qq) * 4 + t) * 2 + cc) * 2 + h;
            const int c = (q[b] >> (4 * rh)) & 15;
            rowmajor[((size_t) n * K + k) >> 1] |= (uint8_t) (c << (4 * (k & 1)));
        }
}

void orc_pack_u4(const uint8_t* rowmajor, int N, int K, uint8_t* q)
{
    const int KB = K / 64;
    memset(q, 0, (size_t) N * K / 2);
    for (int n = 0; n < N; ++n)
        for (int k = 0; k < K; ++k)
        {
            const int gr = n / 64, s = (n % 64) / 16, rh = (n % 16) / 8, g = n % 8;
            const int kb = k / 64, t = (k % 64) / 16, h = (k % 16) / 8, qq = (k % 8) / 2, cc = k % 2;
            const size_t b = ((((((size_t) (gr * KB + kb) * 4 + s) * 8 + g) * 4 + qq) * 4 + t) * 2 + cc) * 2 + h;
            const int c = (rowmajor[((size_t) n * K + k) >> 1] >> (4 * (k & 1))) & 15;
            q[b] |= (uint8_t) (c << (4 * rh));
        }
}

// q8_0 round trip of n values (n % 32 == 0): what the engine's activations look like after quant_group.
void orc_q8_roundtrip(const float* v, int n, float* out)
{
    for (int i = 0; i < n; i += 32)
    {
        int8_t q[32]; float s;
        quant_group32(v + i, q, &s);
        for (int k = 0; k < 32; ++k) out[i + k] = (float) q[k] * s;
    }
}

// One engine job (cpuband.cpp:153-221): R <= 8 rows, selections sel[R][topk] (global ids; only ids in [lo, lo + n)
// count), weights rw fp16. out[R][H] fp32 is overwritten. mode 0 = the reference arithmetic (int8 activations),
// mode 1 = exact activations with double accumulation. If shared != nullptr it is appended as a last pick that every
// row takes with weight 1.
static void job(int H, int I, int G_, int R, int topk, const uint16_t* x, const int64_t* sel, const uint16_t* rw, int lo, int n,
                const orc_expert* ex, const orc_expert* shared, int mode, float* out)
{
    const int GH = G_ ? G_ : H, GI = G_ ? G_ : I;      // scale group of the gate/up matrices (K = H) and of down (K = I)
    const int MAXP = R * topk + 1;
    std::vector<int> pick; pick.reserve(MAXP);
    std::vector<float> wgt((size_t) MAXP * R, 0.f);
    for (int i = 0; i < R * topk; ++i)
    {
        const int64_t e = sel[i] - lo;
        if (e < 0 || e >= n) continue;
        size_t j = 0;
        while (j < pick.size() && pick[j] != (int) e) ++j;
        if (j == pick.size()) pick.push_back((int) e);
        wgt[j * R + i / topk] += h2f(rw[i]);
    }
    const int NPR = (int) pick.size();          // routed picks
    const int NP = NPR + (shared ? 1 : 0);
    std::vector<std::vector<int>> rows(NP);
    for (int p = 0; p < NPR; ++p)
        for (int r = 0; r < R; ++r) if (wgt[(size_t) p * R + r] != 0.f) rows[p].push_back(r);
    if (shared) { for (int r = 0; r < R; ++r) { rows[NPR].push_back(r); wgt[(size_t) NPR * R + r] = 1.f; } }
    auto expert = [&](int p) -> const orc_expert& { return p < NPR ? ex[pick[p]] : *shared; };

    if (NP == 0) { memset(out, 0, (size_t) R * H * 4); return; }

    if (mode == 0)
    {
        std::vector<int8_t> xq((size_t) R * H); std::vector<float> xg((size_t) R * H / 32);
        for (int gi = 0; gi < R * H / 32; ++gi)
        {
            float v[32];
            for (int k = 0; k < 32; ++k) v[k] = h2f(x[(size_t) gi * 32 + k]);
            quant_group32(v, xq.data() + (size_t) gi * 32, xg.data() + gi);
        }
        std::vector<float> gy((size_t) NP * R * I), uy((size_t) NP * R * I);
        #pragma omp parallel for schedule(static) collapse(2)
        for (int p = 0; p < NP; ++p)
            for (int nn = 0; nn < I; ++nn)
            {
                const orc_expert& E = expert(p);
                for (size_t j = 0; j < rows[p].size(); ++j)
                {
                    const int r = rows[p][j];
                    gy[((size_t) p * R + j) * I + nn] = row_dot_q8(E.g + (size_t) nn * H / 2, E.gs + nn, I, H, GH, &xq[(size_t) r * H], &xg[(size_t) r * H / 32]);
                    uy[((size_t) p * R + j) * I + nn] = row_dot_q8(E.u + (size_t) nn * H / 2, E.us + nn, I, H, GH, &xq[(size_t) r * H], &xg[(size_t) r * H / 32]);
                }
            }
        std::vector<int8_t> aq((size_t) NP * R * I); std::vector<float> ag((size_t) NP * R * I / 32);
        for (int p = 0; p < NP; ++p)
            for (size_t j = 0; j < rows[p].size(); ++j)
            {
                const float wt = wgt[(size_t) p * R + rows[p][j]];
                for (int k0 = 0; k0 < I; k0 += 32)
                {
                    float v[32];
                    for (int k = 0; k < 32; ++k)
                    {
                        const float gg = gy[((size_t) p * R + j) * I + k0 + k];
                        v[k] = gg / (1.f + expf(-gg)) * uy[((size_t) p * R + j) * I + k0 + k] * wt;
                    }
                    quant_group32(v, &aq[((size_t) p * R + j) * I + k0], &ag[(((size_t) p * R + j) * I + k0) / 32]);
                }
            }
        #pragma omp parallel for schedule(static)
        for (int nn = 0; nn < H; ++nn)
        {
            float tmp[8];
            for (int r = 0; r < R; ++r) tmp[r] = 0.f;
            for (int p = 0; p < NP; ++p)
            {
                const orc_expert& E = expert(p);
                for (size_t j = 0; j < rows[p].size(); ++j)
                    tmp[rows[p][j]] += row_dot_q8(E.d + (size_t) nn * I / 2, E.ds + nn, H, I, GI, &aq[((size_t) p * R + j) * I], &ag[((size_t) p * R + j) * I / 32]);
            }
            for (int r = 0; r < R; ++r) out[(size_t) r * H + nn] = tmp[r];
        }
    }
    else
    {
        std::vector<double> xd((size_t) R * H);
        for (size_t i = 0; i < xd.size(); ++i) xd[i] = (double) h2f(x[i]);
        std::vector<double> act((size_t) NP * R * I);
        #pragma omp parallel for schedule(static) collapse(2)
        for (int p = 0; p < NP; ++p)
            for (int nn = 0; nn < I; ++nn)
            {
                const orc_expert& E = expert(p);
                for (size_t j = 0; j < rows[p].size(); ++j)
                {
                    const int r = rows[p][j];
                    const double gg = row_dot_exact(E.g + (size_t) nn * H / 2, E.gs + nn, I, H, GH, &xd[(size_t) r * H]);
                    const double uu = row_dot_exact(E.u + (size_t) nn * H / 2, E.us + nn, I, H, GH, &xd[(size_t) r * H]);
                    act[((size_t) p * R + j) * I + nn] = gg / (1.0 + exp(-gg)) * uu * (double) wgt[(size_t) p * R + r];
                }
            }
        #pragma omp parallel for schedule(static)
        for (int nn = 0; nn < H; ++nn)
        {
            double tmp[8];
            for (int r = 0; r < R; ++r) tmp[r] = 0.0;
            for (int p = 0; p < NP; ++p)
            {
                const orc_expert& E = expert(p);
                for (size_t j = 0; j < rows[p].size(); ++j)
                    tmp[rows[p][j]] += row_dot_exact(E.d + (size_t) nn * I / 2, E.ds + nn, H, I, GI, &act[((size_t) p * R + j) * I]);
            }
            for (int r = 0; r < R; ++r) out[(size_t) r * H + nn] = (float) tmp[r];
        }
    }
}

// Any number of rows: independent jobs of <= 8 consecutive rows (the reference acknowledges larger jobs without computing
// them, cpuband.cpp:7,172, and its caller cuts 9..64 rows into 8-row calls, tier_split.py:346-354).
int orc_moe_forward(int H, int I, int G, int R, int topk, const uint16_t* x, const int64_t* sel, const uint16_t* rw, int lo, int n,
                    const orc_expert* ex, const orc_expert* shared, int mode, float* out)
{
    if (H % 64 || I % 64 || G < 0 || G % 32 || (G && (H % G || I % G)) || topk < 1 || R < 0) return 1;
    for (int r0 = 0; r0 < R; r0 += 8)
    {
        const int rr = R - r0 < 8 ? R - r0 : 8;
        job(H, I, G, rr, topk, x + (size_t) r0 * H, sel + (size_t) r0 * topk, rw + (size_t) r0 * topk, lo, n, ex, shared, mode,
            out + (size_t) r0 * H);
    }
    return 0;
}

int orc_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// ---------------------------------------------------------------------------------------------------------------------
// Router (exl3_router.py:21-131 semantics). Every operation is a single correctly rounded IEEE operation in a stated
// order so that the CUDA router, written with the same operations, selects the same experts bit for bit.
//   logit[r][e]: 32 partial sums; partial L runs over columns i*256 + L*8 + j (i outer, j = 0..7 inner) with one fused
//                multiply-add per column; then five butterfly steps p[L] = p[L] + p[L ^ o], o = 16, 8, 4, 2, 1.
//   act = 1 / (1 + exp(-logit)) with the exp below; key = act + bias[e]; top-k by key descending, index ascending;
//   rw = fp16_rn(act * scale / (sum_of_selected_acts_in_selection_order + 1e-20)).
float orc_det_expf(float x)
{
    x = fminf(fmaxf(x, -87.f), 88.f);
    const float t = x * 1.44269504088896341f;
    const float n = rintf(t);
    float r = fmaf(n, -0.693145751953125f, x);
    r = fmaf(n, -1.42860682030941723212e-6f, r);
    float p = 1.9875691500e-4f;
    p = fmaf(p, r, 1.3981999507e-3f);
    p = fmaf(p, r, 8.3334519073e-3f);
    p = fmaf(p, r, 4.1665795894e-2f);
    p = fmaf(p, r, 1.6666665459e-1f);
    p = fmaf(p, r, 5.0000001201e-1f);
    p = fmaf(p, r * r, r);
    p = p + 1.f;
    const int32_t bits = ((int32_t) n + 127) << 23;
    float sc; memcpy(&sc, &bits, 4);
    return p * sc;
}

// x [R][K] and wt [E][K] as raw 16-bit words, fp16 (is_bf16 = 0) or bf16 (1); bias may be null.
int orc_router(const uint16_t* x, int x_bf16, const uint16_t* wt, int w_bf16, const float* bias, int R, int K, int E, int topk,
               float scale, int64_t* sel, uint16_t* rw, float* logits_out)
{
    if (K % 256 || topk > E || topk > 64) return 1;
    auto widen = [](uint16_t v, int bf) -> float {
        if (bf) { uint32_t u = (uint32_t) v << 16; float f; memcpy(&f, &u, 4); return f; }
        return h2f(v);
    };
    std::vector<float> wf((size_t) E * K);
    for (size_t i = 0; i < wf.size(); ++i) wf[i] = widen(wt[i], w_bf16);
    #pragma omp parallel for schedule(static)
    for (int r = 0; r < R; ++r)
    {
        std::vector<float> xr(K), act(E); std::vector<uint32_t> key(E);
        for (int k = 0; k < K; ++k) xr[k] = widen(x[(size_t) r * K + k], x_bf16);
        for (int e = 0; e < E; ++e)
        {
            float p[32];
            const float* w = &wf[(size_t) e * K];
            for (int L = 0; L < 32; ++L)
            {
                float a = 0.f;
                for (int i = 0; i < K / 256; ++i)
                    for (int j = 0; j < 8; ++j) { const int k = i * 256 + L * 8 + j; a = fmaf(xr[k], w[k], a); }
                p[L] = a;
            }
            for (int o = 16; o; o >>= 1)
            {
                float q[32];
                for (int L = 0; L < 32; ++L) q[L] = p[L] + p[L ^ o];
                memcpy(p, q, sizeof(p));
            }
            const float l = p[0];
            if (logits_out) logits_out[(size_t) r * E + e] = l;
            act[e] = 1.f / (1.f + orc_det_expf(-l));
            const float kf = act[e] + (bias ? bias[e] : 0.f);
            uint32_t u; memcpy(&u, &kf, 4);
            key[e] = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
        }
        float sum = 0.f; int ids[64]; float ws[64];
        for (int k = 0; k < topk; ++k)
        {
            int best = 0; uint32_t bk = 0;
            for (int e = 0; e < E; ++e) if (key[e] > bk) { best = e; bk = key[e]; }
            ids[k] = best; ws[k] = act[best]; sum += act[best]; key[best] = 0u;
        }
        for (int k = 0; k < topk; ++k)
        {
            sel[(size_t) r * topk + k] = ids[k];
            rw[(size_t) r * topk + k] = f2h(ws[k] * scale / (sum + 1e-20f));
        }
    }
    return 0;
}

// ---------------------------------------------------------------------------------------------------------------------
// Prefill permutation (tier_split.py:404-412): stable sort of the flattened selection by expert id.
// order[p] = flat pick index, tok = order / topk, eid = sel.flat[order], wt = rw.flat[order] (fp32), counts[E].
void orc_permute(const int64_t* sel, const uint16_t* rw, int R, int topk, int E, int32_t* order, int32_t* tok, int32_t* eid,
                 float* wt, int32_t* counts)
{
    const int np = R * topk;
    std::vector<int64_t> start(E + 1, 0);
    for (int e = 0; e < E; ++e) counts[e] = 0;
    for (int i = 0; i < np; ++i) counts[sel[i]]++;
    for (int e = 0; e < E; ++e) start[e + 1] = start[e] + counts[e];
    std::vector<int64_t> cur(start.begin(), start.end() - 1);
    for (int i = 0; i < np; ++i)
    {
        const int64_t p = cur[sel[i]]++;
        order[p] = i; tok[p] = i / topk; eid[p] = (int32_t) sel[i]; wt[p] = h2f(rw[i]);
    }
}

// Row blocks of one pick group (rtx_split.py:236-255 with npos >= the number of picks): experts without picks emit no
// block; an expert's picks are cut into blocks of <= bm picks, near-equal sizes when balance != 0. rbt [nrb][4] =
// {expert, first pick, picks, 0}. Returns nrb (rbt may be null to count only).
int orc_row_blocks(const int32_t* counts, int E, int bm, int balance, int32_t* rbt)
{
    int nrb = 0; int64_t first = 0;
    for (int e = 0; e < E; ++e)
    {
        const int c = counts[e];
        const int nb = (c + bm - 1) / bm;
        for (int k = 0; k < nb; ++k)
        {
            int rows, start;
            if (balance) { const int base = c / nb, extra = c % nb; rows = base + (k < extra ? 1 : 0); start = k * base + (k < extra ? k : extra); }
            else { rows = c - bm * k < bm ? c - bm * k : bm; start = bm * k; }
            if (rbt) { rbt[4 * nrb + 0] = e; rbt[4 * nrb + 1] = (int32_t) (first + start); rbt[4 * nrb + 2] = rows; rbt[4 * nrb + 3] = 0; }
            ++nrb;
        }
        first += c;
    }
    return nrb;
}

}  // extern "C"

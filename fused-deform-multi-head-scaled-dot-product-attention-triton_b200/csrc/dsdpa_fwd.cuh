// Forward kernel: bilinear sampling of K and V fused with online-softmax attention.
//
// Replaces the reference's _fwd_kernel (ops/triton.py:27-194) and the coordinate scaling
// its host code does before the launch (ops/triton.py:381-383); results follow
// ops/torch.py:5-28 (per-corner zero padding).
//
// Work split.  A CTA owns one (batch, head) and a tile of its queries (query view and
// pixel flattened).  Inside a warp, a group of G lanes owns one query at a time and
// holds a 16-byte slice of every row per lane, so that one gathered row is one
// conflict-free 128-bit shared-memory (or read-only global) load per lane.  Each group
// carries NQ queries ("slots") through the loop over key views, their online-softmax
// state (running max, sum and the D-wide accumulator slice) living in registers.
//
// K/V maps.  STAGED: the K and V maps of the current key view ([L, D] each) are copied
// into shared memory with 1-D bulk copies (cp.async.bulk, completion on an mbarrier),
// double-buffered when two views fit.  Otherwise rows are gathered from L2/L1 with
// ld.global.nc.
//
// Arithmetic is fp32 throughout, two lanes at a time (fma.rn.f32x2) where the data
// comes in pairs.
#pragma once

#include "dsdpa_common.cuh"

// samples handled per iteration of the forward kernel's inner loop
#ifndef DSDPA_FWD_UNROLL
#define DSDPA_FWD_UNROLL 4
#endif
// the same for the variant that gathers from L1/L2 (more CTAs per SM, fewer registers each)
#ifndef DSDPA_FWD_UNROLL_L2
#define DSDPA_FWD_UNROLL_L2 4
#endif

namespace dsdpa {

template <int N> struct IntC { static constexpr int value = N; };   // a compile-time int as an argument

struct FwdParams {
    const void* q;
    const void* k;
    const void* v;
    const float* coords;
    void* out;
    void* out_mirror;    // optional second destination of out (may be another GPU's memory)
    float* lse;
    int B, V, Hh, W, H, L, S;
    float scale2;        // sm_scale * log2(e)
    float hw, hh;        // (W-1)/2 and (H-1)/2
    int tiles;           // tiles per (batch, head)
    int q_per_tile;      // queries per tile
    int nstage;          // STAGED: number of map buffers (1 or 2)
    unsigned map_bytes;  // bytes of one [L, D] map
    int* err;            // device error word
};

// Per-warp scratch that hands the decoded corners of 32 samples from the lane that
// decoded them to the group that consumes them: 32 weight records, then 32 pixel records.
constexpr int kRecBytesPerWarp = 32 * 16 * 2;

// Slot of the record of sample i (0..G-1) of group g inside the per-warp scratch.
// The NG records one step reads are contiguous (conflict-free broadcast reads), and
// the rotation by i/2 spreads the G records a group writes at once over all banks.
template <int G, int NG>
__device__ __forceinline__ uint32_t rec_slot(int i, int g) {
    if constexpr (NG == 4) return (uint32_t)(i * NG + ((g + (i >> 1)) & 3));
    else return (uint32_t)(i * NG + g);
}

template <typename T, int D, bool STAGED>
struct MapReader {
    using RC = RowCfg<T, D>;
    // STAGED: base is a shared-window address; else a global pointer.
    uint32_t sbase;
    const char* gbase;
    int npix;      // pixels per map and the error word, looked at by the checked build only
    int* err;
    __device__ __forceinline__ uint4 load(int pix, int vec) const {
        if (!in_range(pix, npix, err) || !in_range(vec, RC::VEC, err)) return make_uint4(0, 0, 0, 0);
        if constexpr (STAGED) {
            return lds128(sbase + (uint32_t)pix * RC::ROWB + (uint32_t)vec * 16u);
        } else {
            return ldg128_nc(gbase + (size_t)pix * RC::ROWB + (size_t)vec * 16u);
        }
    }
};

// k~ or v~ slice of this lane: sum over the four corners of w_c * row_c, as EPL/2 pairs.
template <typename T, int D, bool STAGED>
__device__ __forceinline__ void gather_interp(const MapReader<T, D, STAGED>& map, const int (&pix)[4],
                                              const float2 (&w2)[4], int li, float2 (&dst)[RowCfg<T, D>::EPL / 2]) {
    using RC = RowCfg<T, D>;
    constexpr int HV = RC::EPV / 2;  // pairs per 16-byte vector
    uint4 raw[4][RC::CH];
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int ch = 0; ch < RC::CH; ++ch) raw[c][ch] = map.load(pix[c], ch * RC::G + li);
#pragma unroll
    for (int ch = 0; ch < RC::CH; ++ch) {
        float2 f[4][HV];
#pragma unroll
        for (int c = 0; c < 4; ++c) unpack16_pairs(raw[c][ch], f[c], (T*)nullptr);
#pragma unroll
        for (int e = 0; e < HV; ++e) {
            float2 a = __fmul2_rn(w2[3], f[3][e]);
            a = __ffma2_rn(w2[2], f[2][e], a);
            a = __ffma2_rn(w2[1], f[1][e], a);
            dst[ch * HV + e] = __ffma2_rn(w2[0], f[0][e], a);
        }
    }
}

// 16-bit storage: this lane's parts d[c] of the four corner dots qv . row_c of one sample, taken
// straight from the stored rows with the mixed-precision fma (no unpack).  `qv` holds the stored
// 16-bit query-side row (q or dout), unscaled.
template <typename T, int D, bool STAGED>
__device__ __forceinline__ void corner_dots16(const MapReader<T, D, STAGED>& map, const int (&pix)[4], int li,
                                              const uint4 (&qv)[RowCfg<T, D>::CH], float (&d)[4]) {
    using RC = RowCfg<T, D>;
    uint4 raw[4][RC::CH];
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int ch = 0; ch < RC::CH; ++ch) raw[c][ch] = map.load(pix[c], ch * RC::G + li);
#pragma unroll
    for (int c = 0; c < 4; ++c) d[c] = 0.0f;
#pragma unroll
    for (int ch = 0; ch < RC::CH; ++ch)
#pragma unroll
        for (int c = 0; c < 4; ++c) d[c] = dot16<T>(qv[ch], raw[c][ch], d[c]);
}

// ... and this lane's part of sum_c w_c (qv . row_c): no interpolated row is ever formed.
template <typename T, int D, bool STAGED>
__device__ __forceinline__ float corner_weighted_dot16(const MapReader<T, D, STAGED>& map, const int (&pix)[4],
                                                       const float2 (&w2)[4], int li,
                                                       const uint4 (&qv)[RowCfg<T, D>::CH]) {
    float d[4];
    corner_dots16<T, D, STAGED>(map, pix, li, qv, d);
    return fmaf(w2[0].x, d[0], fmaf(w2[1].x, d[1], fmaf(w2[2].x, d[2], w2[3].x * d[3])));
}

// Decode the sample of this lane and publish its record for the step that consumes it.
template <int G, int NG>
__device__ __forceinline__ void publish_record(const float2* cptr, int s, int S, int W, int H, float hw, float hh,
                                               uint32_t rec_w, uint32_t rec_p, int li, int g) {
    float2 c = make_float2(0.0f, 0.0f);
    if (s < S) c = __ldg(cptr + s);
    Corners cr;
    float fx, fy;
    decode_corners(c.x, c.y, W, H, hw, hh, cr, fx, fy);
    const uint32_t r = rec_slot<G, NG>(li, g) * 16u;
    sts128(rec_w + r, make_uint4(__float_as_uint(cr.w[0]), __float_as_uint(cr.w[1]), __float_as_uint(cr.w[2]),
                                 __float_as_uint(cr.w[3])));
    sts128(rec_p + r, make_uint4((uint32_t)cr.pix[0], (uint32_t)cr.pix[1], (uint32_t)cr.pix[2], (uint32_t)cr.pix[3]));
}

// Record for the coordinate gradient.  The weight plane holds the ONE-dimensional weights
// {wx0, wx1, wy0, wy1} = {1-fx, fx, 1-fy, fy}, each zeroed when its column / row lies outside the
// map (the four corner weights are their products).  Whether a column / row is inside cannot
// be read off a weight (fx may be exactly 0 for an inside column), so the four flags travel
// in the top bits of the first pixel index: bit 28 column x0, 29 column x1, 30 row y0, 31 row y1.
constexpr uint32_t kPixMask = 0x0fffffffu;

template <int G, int NG>
__device__ __forceinline__ void publish_record_dc(const float2* cptr, int s, int S, int W, int H, float hw, float hh,
                                                  uint32_t rec_w, uint32_t rec_p, int li, int g) {
    float2 c = make_float2(0.0f, 0.0f);
    if (s < S) c = __ldg(cptr + s);
    const float x = unnormalize(c.x, hw), y = unnormalize(c.y, hh);
    const float xf = floorf(x), yf = floorf(y);
    float fx = x - xf, fy = y - yf;
    const bool xr = (xf >= -2.0f) && (xf <= (float)W + 1.0f), yr = (yf >= -2.0f) && (yf <= (float)H + 1.0f);
    const int x0 = xr ? (int)xf : -2, y0 = yr ? (int)yf : -2;
    if (!xr) fx = 0.0f;
    if (!yr) fy = 0.0f;
    const int x1 = x0 + 1, y1 = y0 + 1;
    const bool vx0 = x0 >= 0 && x0 < W, vx1 = x1 >= 0 && x1 < W;
    const bool vy0 = y0 >= 0 && y0 < H, vy1 = y1 >= 0 && y1 < H;
    const float wx0 = vx0 ? 1.0f - fx : 0.0f, wx1 = vx1 ? fx : 0.0f;
    const float wy0 = vy0 ? 1.0f - fy : 0.0f, wy1 = vy1 ? fy : 0.0f;
    const int x0c = min(max(x0, 0), W - 1), x1c = min(max(x1, 0), W - 1);
    const int y0c = min(max(y0, 0), H - 1), y1c = min(max(y1, 0), H - 1);
    const uint32_t flags = (vx0 ? 1u : 0u) | (vx1 ? 2u : 0u) | (vy0 ? 4u : 0u) | (vy1 ? 8u : 0u);
    const uint32_t r = rec_slot<G, NG>(li, g) * 16u;
    sts128(rec_w + r, make_uint4(__float_as_uint(wx0), __float_as_uint(wx1), __float_as_uint(wy0), __float_as_uint(wy1)));
    sts128(rec_p + r, make_uint4((uint32_t)(y0c * W + x0c) | (flags << 28), (uint32_t)(y0c * W + x1c),
                                 (uint32_t)(y1c * W + x0c), (uint32_t)(y1c * W + x1c)));
}

// The four corner rows of a sample against a query-side vector `qv` (q or dout):
// dots[c] = partial (this lane's slice) of qv . row_c, as a pair to be summed, and, if
// WANT_INTERP, interp = sum_c w_c row_c.
template <typename T, int D, bool STAGED, bool WANT_INTERP>
__device__ __forceinline__ void corner_dots(const MapReader<T, D, STAGED>& map, const int (&pix)[4], const float2 (&w2)[4],
                                            int li, const float2 (&qv)[RowCfg<T, D>::EPL / 2],
                                            float2 (&interp)[RowCfg<T, D>::EPL / 2], float2 (&dots)[4]) {
    using RC = RowCfg<T, D>;
    constexpr int HV = RC::EPV / 2;
    uint4 raw[4][RC::CH];
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int ch = 0; ch < RC::CH; ++ch) raw[c][ch] = map.load(pix[c], ch * RC::G + li);
#pragma unroll
    for (int c = 0; c < 4; ++c) dots[c] = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int ch = 0; ch < RC::CH; ++ch) {
        float2 f[4][HV];
#pragma unroll
        for (int c = 0; c < 4; ++c) unpack16_pairs(raw[c][ch], f[c], (T*)nullptr);
#pragma unroll
        for (int e = 0; e < HV; ++e) {
#pragma unroll
            for (int c = 0; c < 4; ++c) dots[c] = __ffma2_rn(qv[ch * HV + e], f[c][e], dots[c]);
            if constexpr (WANT_INTERP) {
                float2 a = __fmul2_rn(w2[3], f[3][e]);
                a = __ffma2_rn(w2[2], f[2][e], a);
                a = __ffma2_rn(w2[1], f[1][e], a);
                interp[ch * HV + e] = __ffma2_rn(w2[0], f[0][e], a);
            }
        }
    }
}

// TAILS: the sample count per key view is not a multiple of the batch size (or a group's chunk of
// samples is smaller than a batch): what is left after the whole batches is taken in twos and
// ones.  Without it every chunk is whole batches and that code is left out, which keeps the
// common case's inner loop as tight as the compiler makes it on its own.
template <typename T, int D, int NQ, bool STAGED, int MAXT, int MINB, bool RW = false, bool TAILS = false>
__global__ void __launch_bounds__(MAXT, MINB) fwd_kernel(const FwdParams p) {
    static_assert(!RW || sizeof(T) == 2, "rounded weights are a 16-bit storage option");
    using RC = RowCfg<T, D>;
    constexpr int G = RC::G, NG = RC::NG, EPL = RC::EPL, CH = RC::CH, EPV = RC::EPV, ROWB = RC::ROWB;
    constexpr int HP = EPL / 2;  // fp32 pairs per lane
    extern __shared__ __align__(128) unsigned char smem[];

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int g = lane / G, li = lane % G;
    const int bh = blockIdx.x / p.tiles, tile = blockIdx.x - bh * p.tiles;
    const int b = bh / p.Hh, h = bh - b * p.Hh;
    const int VL = p.V * p.L;
    const int q0 = tile * p.q_per_tile;
    const int qend = min(q0 + p.q_per_tile, VL);
    const int slot_stride = nw * NG;

    const uint32_t smem0 = smem_addr(smem);
    const uint32_t maps_bytes_all = STAGED ? (uint32_t)p.nstage * 2u * p.map_bytes : 0u;
    const uint32_t rec_w = smem0 + maps_bytes_all + (uint32_t)warp * kRecBytesPerWarp;
    const uint32_t rec_p = rec_w + 32 * 16;
    const uint32_t bar0 = smem0 + maps_bytes_all + (uint32_t)nw * kRecBytesPerWarp;

    const size_t map_stride_view = (size_t)p.Hh * p.map_bytes;  // bytes between views of one head
    const char* kmaps = (const char*)p.k + ((size_t)b * p.V * p.Hh + h) * p.map_bytes;
    const char* vmaps = (const char*)p.v + ((size_t)b * p.V * p.Hh + h) * p.map_bytes;

    if constexpr (STAGED) {
        if (threadIdx.x == 0) {
            // per stage buffer: K's barrier, then V's
            mbar_init(bar0, 1);
            mbar_init(bar0 + 8, 1);
            mbar_init(bar0 + 16, 1);
            mbar_init(bar0 + 24, 1);
            fence_mbar_init();
            fence_proxy_async();
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            stage_maps(smem0, kmaps, vmaps, p.map_bytes, bar0);
        }
    }

    float m_run[NQ], l_run[NQ];
    float2 acc[NQ][HP];
#pragma unroll
    for (int j = 0; j < NQ; ++j) {
        m_run[j] = -INFINITY;
        l_run[j] = 0.0f;
#pragma unroll
        for (int e = 0; e < HP; ++e) acc[j][e] = make_float2(0.0f, 0.0f);
    }

    for (int vk = 0; vk < p.V; ++vk) {
        MapReader<T, D, STAGED> kmap, vmap;
        kmap.npix = vmap.npix = p.L;
        kmap.err = vmap.err = p.err;
        bool ok = true;
        // STAGED: the V map's barrier of this key view, waited for right behind K's (a wait that
        // runs out is recorded and ends the CTA at the view's end)
        uint32_t bar_v = 0;
        unsigned par_v = 0;
        bool v_ready = true;
        auto v_wait = [&]() {
            if constexpr (STAGED) {
                if (!v_ready) {
                    if (!mbar_wait_bounded(bar_v, par_v, p.err)) ok = false;
                    v_ready = true;
                }
            }
        };
        if constexpr (STAGED) {
            const int stage = p.nstage == 2 ? (vk & 1) : 0;
            if (p.nstage == 2 && vk + 1 < p.V && threadIdx.x == 0) {
                const uint32_t bar = bar0 + 16u * (uint32_t)((vk + 1) & 1);
                const uint32_t dst = smem0 + (uint32_t)((vk + 1) & 1) * 2u * p.map_bytes;
                stage_maps(dst, kmaps + (size_t)(vk + 1) * map_stride_view, vmaps + (size_t)(vk + 1) * map_stride_view,
                           p.map_bytes, bar);
            }
            const unsigned parity = p.nstage == 2 ? ((unsigned)(vk >> 1) & 1u) : ((unsigned)vk & 1u);
            // K first, then V (v_wait below)
            bar_v = bar0 + 16u * (uint32_t)stage + 8u;
            par_v = parity;
            v_ready = false;
            ok = mbar_wait_bounded(bar0 + 16u * (uint32_t)stage, parity, p.err);
            ok = __all_sync(0xffffffffu, ok);
            kmap.sbase = smem0 + (uint32_t)stage * 2u * p.map_bytes;
            vmap.sbase = kmap.sbase + p.map_bytes;
            kmap.gbase = vmap.gbase = nullptr;
        } else {
            kmap.gbase = kmaps + (size_t)vk * map_stride_view;
            vmap.gbase = vmaps + (size_t)vk * map_stride_view;
            kmap.sbase = vmap.sbase = 0;
        }

        // (Waiting for V only where the first V row is needed was measured slower, here and in the
        // backward's first pass: the test in front of the V gathers keeps the compiler from moving
        // their loads up into the arithmetic before them.)
        v_wait();
        if (ok) {
#pragma unroll
            for (int j = 0; j < NQ; ++j) {
                const int qslot = q0 + j * slot_stride + warp * NG + g;
                // warps whose every slot is past the tile end have nothing to do
                if (q0 + j * slot_stride + warp * NG >= qend) continue;
                const int qi = min(qslot, qend - 1);  // surplus groups redo the last query; never stored
                const int vq = qi / p.L, l = qi - vq * p.L;
                const size_t qrow = (((size_t)b * p.V + vq) * p.Hh + h) * p.L + l;
                // fp32 storage: q in registers as fp32 pairs with the scale folded in; 16-bit storage: the
                // stored row as it is (the logit's corner dots use the mixed-precision fma, the scale
                // is applied to the reduced logit)
                constexpr bool NARROW = sizeof(T) == 2;
                float2 qf[HP];
                uint4 qraw[CH];
#pragma unroll
                for (int ch = 0; ch < CH; ++ch) {
                    qraw[ch] = ldg128_nc((const char*)p.q + qrow * ROWB + (size_t)(ch * G + li) * 16);
                    if constexpr (!NARROW) {
                        float2 f[EPV / 2];
                        unpack16_pairs(qraw[ch], f, (T*)nullptr);
#pragma unroll
                        for (int e = 0; e < EPV / 2; ++e)
                            qf[ch * (EPV / 2) + e] = make_float2(f[e].x * p.scale2, f[e].y * p.scale2);
                    }
                }
                const float2* cptr = reinterpret_cast<const float2*>(p.coords) +
                                     ((((size_t)b * p.V + vq) * p.L + l) * p.V + vk) * (size_t)p.S;
                float m = m_run[j], lsum = l_run[j];
                for (int s0 = 0; s0 < p.S; s0 += G) {
                    publish_record<G, NG>(cptr, s0 + li, p.S, p.W, p.H, p.hw, p.hh, rec_w, rec_p, li, g);
                    __syncwarp();
                    const int cnt = min(G, p.S - s0);
                    // U samples per iteration: their gathers and dot-product reductions overlap, and
                    // the running maximum is updated once for the batch
                    constexpr int UMAX = STAGED ? DSDPA_FWD_UNROLL : DSDPA_FWD_UNROLL_L2;
                    // samples i .. i+U-1 of the chunk.  TAILS: all of them exist; else samples past the
                    // chunk's end repeat its last one and are masked out of the softmax
                    auto batch = [&](int i, auto u_const) {
                        constexpr int U = decltype(u_const)::value;
                        float2 w2[U][4];
                        int pix[U][4];
#pragma unroll
                        for (int u = 0; u < U; ++u) {
                            const uint32_t r = rec_slot<G, NG>(TAILS ? i + u : min(i + u, cnt - 1), g) * 16u;
                            const uint4 wr = lds128(rec_w + r), pr = lds128(rec_p + r);
                            w2[u][0] = make_float2(__uint_as_float(wr.x), __uint_as_float(wr.x));
                            w2[u][1] = make_float2(__uint_as_float(wr.y), __uint_as_float(wr.y));
                            w2[u][2] = make_float2(__uint_as_float(wr.z), __uint_as_float(wr.z));
                            w2[u][3] = make_float2(__uint_as_float(wr.w), __uint_as_float(wr.w));
                            pix[u][0] = (int)pr.x; pix[u][1] = (int)pr.y; pix[u][2] = (int)pr.z; pix[u][3] = (int)pr.w;
                        }
                        float sc[U];
#pragma unroll
                        for (int u = 0; u < U; ++u) {
                            if constexpr (NARROW) {
                                sc[u] = corner_weighted_dot16<T, D, STAGED>(kmap, pix[u], w2[u], li, qraw);
                            } else {
                                float2 kt[HP];
                                gather_interp<T, D, STAGED>(kmap, pix[u], w2[u], li, kt);
                                float2 part = __fmul2_rn(qf[0], kt[0]);
#pragma unroll
                                for (int e = 1; e < HP; ++e) part = __ffma2_rn(qf[e], kt[e], part);
                                sc[u] = part.x + part.y;
                            }
                        }
#pragma unroll
                        for (int o = G / 2; o > 0; o >>= 1)
#pragma unroll
                            for (int u = 0; u < U; ++u) sc[u] += __shfl_xor_sync(0xffffffffu, sc[u], o);
                        if constexpr (NARROW) {
#pragma unroll
                            for (int u = 0; u < U; ++u) sc[u] *= p.scale2;
                        }
                        float smax = sc[0];
#pragma unroll
                        for (int u = 1; u < U; ++u) {
                            if (!TAILS && i + u >= cnt) sc[u] = -INFINITY;    // same for the whole warp
                            smax = fmaxf(smax, sc[u]);
                        }
                        if (smax > m) {
                            // new running maximum: rescale what has been accumulated so far
                            const float alpha = fast_exp2(m - smax);
                            lsum *= alpha;
                            const float2 a2 = make_float2(alpha, alpha);
#pragma unroll
                            for (int e = 0; e < HP; ++e) acc[j][e] = __fmul2_rn(acc[j][e], a2);
                            m = smax;
                        }
#pragma unroll
                        for (int u = 0; u < U; ++u) {
                            const float pe = fast_exp2(sc[u] - m);
                            lsum += pe;
                            if constexpr (RW) {
                                // (option) acc += sum_c (p*w_c) V_c straight from the stored rows: the
                                // four weights p*w_c are rounded to the storage type (as the probabilities
                                // are before the P.V product of a dense 16-bit attention kernel), products
                                // exact, sums fp32; the normaliser keeps the unrounded p
                                uint16_t s4[4];
                                round_pair16(pe * w2[u][0].x, pe * w2[u][1].x, s4[0], s4[1], (T*)nullptr);
                                round_pair16(pe * w2[u][2].x, pe * w2[u][3].x, s4[2], s4[3], (T*)nullptr);
                                uint4 raw[4][CH];
#pragma unroll
                                for (int c = 0; c < 4; ++c)
#pragma unroll
                                    for (int ch = 0; ch < CH; ++ch) raw[c][ch] = vmap.load(pix[u][c], ch * G + li);
#pragma unroll
                                for (int ch = 0; ch < CH; ++ch)
#pragma unroll
                                    for (int c = 0; c < 4; ++c) axpy16<T>(s4[c], raw[c][ch], &acc[j][ch * (EPV / 2)]);
                            } else {
                                float2 vt[HP];
                                gather_interp<T, D, STAGED>(vmap, pix[u], w2[u], li, vt);
                                const float2 p2 = make_float2(pe, pe);
#pragma unroll
                                for (int e = 0; e < HP; ++e) acc[j][e] = __ffma2_rn(p2, vt[e], acc[j][e]);
                            }
                        }
                    };
                    if constexpr (!TAILS) {
                        for (int i = 0; i < cnt; i += UMAX) batch(i, IntC<UMAX>{});
                    } else {
                        // whole batches, then what is left in twos and ones: no padded work
                        int i = 0;
                        for (; i + UMAX <= cnt; i += UMAX) batch(i, IntC<UMAX>{});
                        if constexpr (UMAX > 2) {
                            for (; i + 2 <= cnt; i += 2) batch(i, IntC<2>{});
                        }
                        if constexpr (UMAX > 1) {
                            for (; i < cnt; ++i) batch(i, IntC<1>{});
                        }
                    }
                    __syncwarp();
                }
                m_run[j] = m;
                l_run[j] = lsum;
            }
        }
        if constexpr (STAGED) {
            // every warp is done with this buffer before it is refilled
            if (__syncthreads_or(ok ? 0 : 1)) return;
            if (p.nstage == 1 && vk + 1 < p.V && threadIdx.x == 0) {
                stage_maps(smem0, kmaps + (size_t)(vk + 1) * map_stride_view, vmaps + (size_t)(vk + 1) * map_stride_view,
                           p.map_bytes, bar0);
            }
        }
    }

#pragma unroll
    for (int j = 0; j < NQ; ++j) {
        const int qi = q0 + j * slot_stride + warp * NG + g;
        if (qi >= qend) continue;
        const int vq = qi / p.L, l = qi - vq * p.L;
        const size_t qrow = (((size_t)b * p.V + vq) * p.Hh + h) * p.L + l;
        const float inv = 1.0f / l_run[j];
#pragma unroll
        for (int ch = 0; ch < CH; ++ch) {
            float f[EPV];
#pragma unroll
            for (int e = 0; e < EPV / 2; ++e) {
                f[2 * e] = acc[j][ch * (EPV / 2) + e].x * inv;
                f[2 * e + 1] = acc[j][ch * (EPV / 2) + e].y * inv;
            }
            const uint4 packed = pack16(f, (T*)nullptr);
            stg128((char*)p.out + qrow * ROWB + (size_t)(ch * G + li) * 16, packed);
            if (p.out_mirror) stg128((char*)p.out_mirror + qrow * ROWB + (size_t)(ch * G + li) * 16, packed);
        }
        if (li == 0) p.lse[qrow] = m_run[j] + log2f(l_run[j]);
    }
}

}  // namespace dsdpa

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
#pragma once

#include "dsdpa_common.cuh"

namespace dsdpa {

struct FwdParams {
    const void* q;
    const void* k;
    const void* v;
    const float* coords;
    void* out;
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
// decoded them to the group that consumes them.
constexpr int kRecBytesPerWarp = 32 * 16 * 2;

template <typename T, int D, bool STAGED>
struct MapReader {
    using RC = RowCfg<T, D>;
    // STAGED: base is a shared-window address; else a global pointer.
    uint32_t sbase;
    const char* gbase;
    __device__ __forceinline__ uint4 load(int pix, int vec) const {
        if constexpr (STAGED) {
            return lds128(sbase + (uint32_t)pix * RC::ROWB + (uint32_t)vec * 16u);
        } else {
            return ldg128_nc(gbase + (size_t)pix * RC::ROWB + (size_t)vec * 16u);
        }
    }
};

// k~ or v~ slice of this lane: sum over the four corners of w_c * row_c.
template <typename T, int D, bool STAGED>
__device__ __forceinline__ void gather_interp(const MapReader<T, D, STAGED>& map, const int (&pix)[4],
                                              const float (&w)[4], int li, float (&dst)[RowCfg<T, D>::EPL]) {
    using RC = RowCfg<T, D>;
    uint4 raw[4][RC::CH];
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int ch = 0; ch < RC::CH; ++ch) raw[c][ch] = map.load(pix[c], ch * RC::G + li);
#pragma unroll
    for (int ch = 0; ch < RC::CH; ++ch) {
        float f[4][RC::EPV];
#pragma unroll
        for (int c = 0; c < 4; ++c) unpack16(raw[c][ch], f[c], (T*)nullptr);
#pragma unroll
        for (int e = 0; e < RC::EPV; ++e)
            dst[ch * RC::EPV + e] = fmaf(w[0], f[0][e], fmaf(w[1], f[1][e], fmaf(w[2], f[2][e], w[3] * f[3][e])));
    }
}

template <typename T, int D, int NQ, bool STAGED, int MAXT, int MINB>
__global__ void __launch_bounds__(MAXT, MINB) fwd_kernel(const FwdParams p) {
    using RC = RowCfg<T, D>;
    constexpr int G = RC::G, NG = RC::NG, EPL = RC::EPL, CH = RC::CH, EPV = RC::EPV, ROWB = RC::ROWB;
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
            mbar_init(bar0, 1);
            mbar_init(bar0 + 8, 1);
            fence_mbar_init();
            fence_proxy_async();
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            mbar_expect_tx(bar0, 2u * p.map_bytes);
            bulk_g2s_chunked(smem0, kmaps, p.map_bytes, bar0);
            bulk_g2s_chunked(smem0 + p.map_bytes, vmaps, p.map_bytes, bar0);
        }
    }

    float m_run[NQ], l_run[NQ], acc[NQ][EPL];
#pragma unroll
    for (int j = 0; j < NQ; ++j) {
        m_run[j] = -INFINITY;
        l_run[j] = 0.0f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[j][e] = 0.0f;
    }

    for (int vk = 0; vk < p.V; ++vk) {
        MapReader<T, D, STAGED> kmap, vmap;
        bool ok = true;
        if constexpr (STAGED) {
            const int stage = p.nstage == 2 ? (vk & 1) : 0;
            if (p.nstage == 2 && vk + 1 < p.V && threadIdx.x == 0) {
                const uint32_t bar = bar0 + 8u * (uint32_t)((vk + 1) & 1);
                const uint32_t dst = smem0 + (uint32_t)((vk + 1) & 1) * 2u * p.map_bytes;
                fence_proxy_async();
                mbar_expect_tx(bar, 2u * p.map_bytes);
                bulk_g2s_chunked(dst, kmaps + (size_t)(vk + 1) * map_stride_view, p.map_bytes, bar);
                bulk_g2s_chunked(dst + p.map_bytes, vmaps + (size_t)(vk + 1) * map_stride_view, p.map_bytes, bar);
            }
            const unsigned parity = p.nstage == 2 ? ((unsigned)(vk >> 1) & 1u) : ((unsigned)vk & 1u);
            ok = mbar_wait_bounded(bar0 + 8u * (uint32_t)stage, parity, p.err);
            ok = __all_sync(0xffffffffu, ok);
            kmap.sbase = smem0 + (uint32_t)stage * 2u * p.map_bytes;
            vmap.sbase = kmap.sbase + p.map_bytes;
            kmap.gbase = vmap.gbase = nullptr;
        } else {
            kmap.gbase = kmaps + (size_t)vk * map_stride_view;
            vmap.gbase = vmaps + (size_t)vk * map_stride_view;
            kmap.sbase = vmap.sbase = 0;
        }

        if (ok) {
#pragma unroll
            for (int j = 0; j < NQ; ++j) {
                const int qslot = q0 + j * slot_stride + warp * NG + g;
                // warps whose every slot is past the tile end have nothing to do
                if (q0 + j * slot_stride + warp * NG >= qend) continue;
                const int qi = min(qslot, qend - 1);  // surplus groups redo the last query; never stored
                const int vq = qi / p.L, l = qi - vq * p.L;
                const size_t qrow = (((size_t)b * p.V + vq) * p.Hh + h) * p.L + l;
                float qf[EPL];
#pragma unroll
                for (int ch = 0; ch < CH; ++ch) {
                    uint4 raw = ldg128_nc((const char*)p.q + qrow * ROWB + (size_t)(ch * G + li) * 16);
                    float f[EPV];
                    unpack16(raw, f, (T*)nullptr);
#pragma unroll
                    for (int e = 0; e < EPV; ++e) qf[ch * EPV + e] = f[e] * p.scale2;
                }
                const float2* cptr = reinterpret_cast<const float2*>(p.coords) +
                                     ((((size_t)b * p.V + vq) * p.L + l) * p.V + vk) * (size_t)p.S;
                float m = m_run[j], lsum = l_run[j];
                for (int s0 = 0; s0 < p.S; s0 += G) {
                    {
                        const int s = s0 + li;
                        float2 c = make_float2(0.0f, 0.0f);
                        if (s < p.S) c = __ldg(cptr + s);
                        Corners cr;
                        float fx, fy;
                        decode_corners(c.x, c.y, p.W, p.H, p.hw, p.hh, cr, fx, fy);
                        const uint32_t r = (uint32_t)(li * NG + g) * 16u;
                        sts128(rec_w + r, make_uint4(__float_as_uint(cr.w[0]), __float_as_uint(cr.w[1]),
                                                     __float_as_uint(cr.w[2]), __float_as_uint(cr.w[3])));
                        sts128(rec_p + r, make_uint4((uint32_t)cr.pix[0], (uint32_t)cr.pix[1],
                                                     (uint32_t)cr.pix[2], (uint32_t)cr.pix[3]));
                    }
                    __syncwarp();
                    const int cnt = min(G, p.S - s0);
#pragma unroll 2
                    for (int i = 0; i < cnt; ++i) {
                        const uint32_t r = (uint32_t)(i * NG + g) * 16u;
                        const uint4 wr = lds128(rec_w + r), pr = lds128(rec_p + r);
                        const float w[4] = { __uint_as_float(wr.x), __uint_as_float(wr.y),
                                             __uint_as_float(wr.z), __uint_as_float(wr.w) };
                        const int pix[4] = { (int)pr.x, (int)pr.y, (int)pr.z, (int)pr.w };
                        float kt[EPL], vt[EPL];
                        gather_interp<T, D, STAGED>(kmap, pix, w, li, kt);
                        gather_interp<T, D, STAGED>(vmap, pix, w, li, vt);
                        float part = 0.0f;
#pragma unroll
                        for (int e = 0; e < EPL; ++e) part = fmaf(qf[e], kt[e], part);
                        const float sc = group_sum<G>(part);
                        const float m_new = fmaxf(m, sc);
                        const float alpha = fast_exp2(m - m_new);
                        const float pe = fast_exp2(sc - m_new);
                        lsum = fmaf(lsum, alpha, pe);
#pragma unroll
                        for (int e = 0; e < EPL; ++e) acc[j][e] = fmaf(pe, vt[e], acc[j][e] * alpha);
                        m = m_new;
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
                fence_proxy_async();
                mbar_expect_tx(bar0, 2u * p.map_bytes);
                bulk_g2s_chunked(smem0, kmaps + (size_t)(vk + 1) * map_stride_view, p.map_bytes, bar0);
                bulk_g2s_chunked(smem0 + p.map_bytes, vmaps + (size_t)(vk + 1) * map_stride_view, p.map_bytes, bar0);
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
            for (int e = 0; e < EPV; ++e) f[e] = acc[j][ch * EPV + e] * inv;
            stg128((char*)p.out + qrow * ROWB + (size_t)(ch * G + li) * 16, pack16(f, (T*)nullptr));
        }
        if (li == 0) p.lse[qrow] = m_run[j] + log2f(l_run[j]);
    }
}

}  // namespace dsdpa

// Backward, one-kernel scatter form.
//
// Replaces the reference's _bwd_preprocess (ops/triton.py:197-215), _bwd_kernel
// (ops/triton.py:219-365) and the K pre-scaling / fp32->storage casts around them
// (ops/triton.py:431-432, 461-462).  Per query-head and sampled key n:
//     p_n  = exp2(scale2 * q.k~_n - lse)                (recomputed, ops/triton.py:330-333)
//     ds_n = p_n * (dout.v~_n - delta),  delta = out.dout
//     dq   = sm_scale * sum_n ds_n k~_n
//     dK[pix_c] += sm_scale * ds_n * w_c * q,   dV[pix_c] += p_n * w_c * dout   (valid corners c)
// with per-corner zero padding as in ops/torch.py:14-15.
//
// Same work split as the forward kernel (a group of G lanes per query, NQ query slots
// per group, K/V maps of the current key view staged in shared memory or gathered from
// L2).  The scatter goes either
//   PRIV:  into fp32 dK/dV maps of the current key view held in shared memory
//          (red.shared.add.f32), flushed once per key view with 16-byte vector
//          reductions (red.global.add.v4.f32), or
//   else:  straight to global memory with red.global.add.v4.f32.
// The global accumulators are fp32 ([B,V,Hh,L,D]); for fp32 storage they are the dk/dv
// outputs themselves.
#pragma once

#include "dsdpa_fwd.cuh"

namespace dsdpa {

struct BwdParams {
    const void* q;
    const void* k;
    const void* v;
    const float* coords;
    const void* out;
    const float* lse;
    const void* dout;
    void* dq;
    void* out_mirror;     // optional: receives a copy of the out rows this kernel reads
    void* dq_mirror;      // optional second destination of dq
    float* dk32;
    float* dv32;
    float* dcoords;
    int B, V, Hh, W, H, L, S;
    float sm_scale, scale2;
    float hw, hh;
    int tiles, q_per_tile, nstage;
    unsigned map_bytes;   // bytes of one [L, D] map in the storage type
    unsigned acc_bytes;   // bytes of one [L, D] fp32 map (PRIV)
    int* err;             // device error word
    // two-pass form: per-sample scalars (sm_scale*ds, p) for the gather pass, laid out
    // [B, Hh, V*tpv tiles, V key views, QB queries, S] as float2
    float2* scal;
    int tpv;              // gather-pass tiles per query view
    int QB;               // queries per gather-pass tile
};

// TWOPASS: no scatter; instead every sample's (sm_scale*ds, p) is written out for the
// gather pass (bwd_gather_kernel) that forms dK/dV without atomics.
// DCOORDS (two-pass form only): additionally d(loss)/d(coords), summed over the heads with
// red.global.add.v2.f32.  With k~ = sum_c w_c K_c and A_c = q.K_c, B_c = dout.V_c the gradient
// w.r.t. the pixel position is  a*(d w_c/dx) A_c + p*(d w_c/dx) B_c  summed over the valid
// corners (a = sm_scale*ds), times (W-1) resp. (H-1) for the normalised coordinate
// (grid_sample backward w.r.t. the grid chained through grid = c*2-1, ops/torch.py:14).
template <typename T, int D, int NQ, bool STAGED, bool PRIV, bool TWOPASS, bool DCOORDS, int MAXT, int MINB>
__global__ void __launch_bounds__(MAXT, MINB) bwd_scatter_kernel(const BwdParams p) {
    static_assert(!PRIV || STAGED, "privatised accumulators live next to staged maps");
    static_assert(!(PRIV && TWOPASS), "the two-pass form has nothing to privatise");
    static_assert(!DCOORDS || TWOPASS, "the coordinate gradient is built into the two-pass form only");
    using RC = RowCfg<T, D>;
    constexpr int G = RC::G, NG = RC::NG, EPL = RC::EPL, CH = RC::CH, EPV = RC::EPV, ROWB = RC::ROWB;
    constexpr int HP = EPL / 2, HV = EPV / 2;  // fp32 pairs per lane / per 16-byte vector
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
    const uint32_t acc_k = smem0 + maps_bytes_all;           // PRIV: fp32 dK map, then dV map
    const uint32_t acc_v = acc_k + p.acc_bytes;
    const uint32_t after_acc = maps_bytes_all + (PRIV ? 2u * p.acc_bytes : 0u);
    const uint32_t rec_w = smem0 + after_acc + (uint32_t)warp * kRecBytesPerWarp;
    const uint32_t rec_p = rec_w + 32 * 16;
    const uint32_t bar0 = smem0 + after_acc + (uint32_t)nw * kRecBytesPerWarp;

    const size_t map_stride_view = (size_t)p.Hh * p.map_bytes;
    const char* kmaps = (const char*)p.k + ((size_t)b * p.V * p.Hh + h) * p.map_bytes;
    const char* vmaps = (const char*)p.v + ((size_t)b * p.V * p.Hh + h) * p.map_bytes;
    const size_t acc_stride_view = (size_t)p.Hh * p.L * D;   // floats between views of one head
    float* dkmaps = p.dk32 + ((size_t)b * p.V * p.Hh + h) * (size_t)p.L * D;
    float* dvmaps = p.dv32 + ((size_t)b * p.V * p.Hh + h) * (size_t)p.L * D;

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
        if constexpr (PRIV) {
            for (uint32_t o = threadIdx.x * 16u; o < 2u * p.acc_bytes; o += blockDim.x * 16u)
                sts128(acc_k + o, make_uint4(0, 0, 0, 0));
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            stage_maps(smem0, kmaps, vmaps, p.map_bytes, bar0);
        }
    }

    // per-slot state that does not depend on the key view
    float2 dq[NQ][HP];
    float lse_q[NQ], delta_q[NQ];
#pragma unroll
    for (int j = 0; j < NQ; ++j) {
#pragma unroll
        for (int e = 0; e < HP; ++e) dq[j][e] = make_float2(0.0f, 0.0f);
        lse_q[j] = 0.0f;
        delta_q[j] = 0.0f;
        if (q0 + j * slot_stride + warp * NG >= qend) continue;
        const int qi = min(q0 + j * slot_stride + warp * NG + g, qend - 1);
        const int vq = qi / p.L, l = qi - vq * p.L;
        const size_t qrow = (((size_t)b * p.V + vq) * p.Hh + h) * p.L + l;
        float part = 0.0f;
#pragma unroll
        for (int ch = 0; ch < CH; ++ch) {
            float fo[EPV], fd[EPV];
            const uint4 oraw = ldg128_nc((const char*)p.out + qrow * ROWB + (size_t)(ch * G + li) * 16);
            unpack16(oraw, fo, (T*)nullptr);
            // (slots past the tile's end repeat its last query: the copy is then the same row again)
            if (p.out_mirror) stg128((char*)p.out_mirror + qrow * ROWB + (size_t)(ch * G + li) * 16, oraw);
            unpack16(ldg128_nc((const char*)p.dout + qrow * ROWB + (size_t)(ch * G + li) * 16), fd, (T*)nullptr);
#pragma unroll
            for (int e = 0; e < EPV; ++e) part = fmaf(fo[e], fd[e], part);
        }
        delta_q[j] = group_sum<G>(part);
        lse_q[j] = __ldg(p.lse + qrow);
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
        float* dkmap = dkmaps + (size_t)vk * acc_stride_view;
        float* dvmap = dvmaps + (size_t)vk * acc_stride_view;

        // (as in the forward: waiting for V only in front of the first V row was measured slower)
        v_wait();
        if (ok) {
#pragma unroll
            for (int j = 0; j < NQ; ++j) {
                if (q0 + j * slot_stride + warp * NG >= qend) continue;
                const int qslot = q0 + j * slot_stride + warp * NG + g;
                const bool live = qslot < qend;       // surplus groups compute but never scatter
                const int qi = min(qslot, qend - 1);
                const int vq = qi / p.L, l = qi - vq * p.L;
                const size_t qrow = (((size_t)b * p.V + vq) * p.Hh + h) * p.L + l;
                float2 qf[HP], dof[HP];
                uint4 doraw[CH];   // the stored dout row (16-bit storage: dout.v~ from corner dots)
#pragma unroll
                for (int ch = 0; ch < CH; ++ch) {
                    float2 f[HV];
                    unpack16_pairs(ldg128_nc((const char*)p.q + qrow * ROWB + (size_t)(ch * G + li) * 16), f, (T*)nullptr);
#pragma unroll
                    for (int e = 0; e < HV; ++e) qf[ch * HV + e] = make_float2(f[e].x * p.scale2, f[e].y * p.scale2);
                    doraw[ch] = ldg128_nc((const char*)p.dout + qrow * ROWB + (size_t)(ch * G + li) * 16);
                    unpack16_pairs(doraw[ch], f, (T*)nullptr);
#pragma unroll
                    for (int e = 0; e < HV; ++e) dof[ch * HV + e] = f[e];
                }
                const float2* cptr = reinterpret_cast<const float2*>(p.coords) +
                                     ((((size_t)b * p.V + vq) * p.L + l) * p.V + vk) * (size_t)p.S;
                const float lse = lse_q[j], delta = delta_q[j];
                float2* scal_row = nullptr;
                if constexpr (TWOPASS) {
                    const int tl = l / p.QB, ql = l - tl * p.QB;
                    const size_t tile = ((size_t)b * p.Hh + h) * (size_t)(p.V * p.tpv) + (size_t)(vq * p.tpv + tl);
                    scal_row = p.scal + ((tile * p.V + vk) * (size_t)p.QB + ql) * (size_t)p.S;
                }
                for (int s0 = 0; s0 < p.S; s0 += G) {
                    float my_a = 0.0f, my_p = 0.0f;  // TWOPASS: scalars of sample s0+li
                    if constexpr (DCOORDS) {
                        publish_record_dc<G, NG>(cptr, s0 + li, p.S, p.W, p.H, p.hw, p.hh, rec_w, rec_p, li, g);
                    } else {
                        publish_record<G, NG>(cptr, s0 + li, p.S, p.W, p.H, p.hw, p.hh, rec_w, rec_p, li, g);
                    }
                    float my_gx = 0.0f, my_gy = 0.0f;  // DCOORDS: gradient of sample s0+li
                    __syncwarp();
                    const int cnt = min(G, p.S - s0);
                    // The common case (two-pass form, no coordinate gradient) takes two samples per
                    // iteration so that their gathers and the four reductions overlap.
                    constexpr bool PAIRS = TWOPASS && !DCOORDS;
                    for (int i = 0; PAIRS && i < cnt; i += 2) {
                        const bool two = i + 1 < cnt;              // same for the whole warp
                        const int ib = two ? i + 1 : i;
                        const uint32_t ra = rec_slot<G, NG>(i, g) * 16u, rb = rec_slot<G, NG>(ib, g) * 16u;
                        const uint4 wa = lds128(rec_w + ra), pa = lds128(rec_p + ra);
                        const uint4 wb = lds128(rec_w + rb), pb = lds128(rec_p + rb);
                        const float2 w2a[4] = { make_float2(__uint_as_float(wa.x), __uint_as_float(wa.x)),
                                                make_float2(__uint_as_float(wa.y), __uint_as_float(wa.y)),
                                                make_float2(__uint_as_float(wa.z), __uint_as_float(wa.z)),
                                                make_float2(__uint_as_float(wa.w), __uint_as_float(wa.w)) };
                        const float2 w2b[4] = { make_float2(__uint_as_float(wb.x), __uint_as_float(wb.x)),
                                                make_float2(__uint_as_float(wb.y), __uint_as_float(wb.y)),
                                                make_float2(__uint_as_float(wb.z), __uint_as_float(wb.z)),
                                                make_float2(__uint_as_float(wb.w), __uint_as_float(wb.w)) };
                        const int pixa[4] = { (int)pa.x, (int)pa.y, (int)pa.z, (int)pa.w };
                        const int pixb[4] = { (int)pb.x, (int)pb.y, (int)pb.z, (int)pb.w };
                        // k~ is needed as a vector (dq accumulates ds*k~); of v~ only dout.v~, which for
                        // 16-bit storage comes from the corner dots of the stored rows (mixed-precision
                        // fma: no unpack, no interpolated row)
                        float2 kta[HP], ktb[HP];
                        gather_interp<T, D, STAGED>(kmap, pixa, w2a, li, kta);
                        gather_interp<T, D, STAGED>(kmap, pixb, w2b, li, ktb);
                        float2 psa = __fmul2_rn(qf[0], kta[0]), psb = __fmul2_rn(qf[0], ktb[0]);
#pragma unroll
                        for (int e = 1; e < HP; ++e) {
                            psa = __ffma2_rn(qf[e], kta[e], psa);
                            psb = __ffma2_rn(qf[e], ktb[e], psb);
                        }
                        float sa = psa.x + psa.y, sb = psb.x + psb.y, da, db;
                        if constexpr (sizeof(T) == 2) {
                            da = corner_weighted_dot16<T, D, STAGED>(vmap, pixa, w2a, li, doraw);
                            db = corner_weighted_dot16<T, D, STAGED>(vmap, pixb, w2b, li, doraw);
                        } else {
                            float2 vta[HP], vtb[HP];
                            gather_interp<T, D, STAGED>(vmap, pixa, w2a, li, vta);
                            gather_interp<T, D, STAGED>(vmap, pixb, w2b, li, vtb);
                            float2 pda = __fmul2_rn(dof[0], vta[0]), pdb = __fmul2_rn(dof[0], vtb[0]);
#pragma unroll
                            for (int e = 1; e < HP; ++e) {
                                pda = __ffma2_rn(dof[e], vta[e], pda);
                                pdb = __ffma2_rn(dof[e], vtb[e], pdb);
                            }
                            da = pda.x + pda.y;
                            db = pdb.x + pdb.y;
                        }
#pragma unroll
                        for (int o = G / 2; o > 0; o >>= 1) {
                            sa += __shfl_xor_sync(0xffffffffu, sa, o);
                            sb += __shfl_xor_sync(0xffffffffu, sb, o);
                            da += __shfl_xor_sync(0xffffffffu, da, o);
                            db += __shfl_xor_sync(0xffffffffu, db, o);
                        }
                        const float pea = fast_exp2(sa - lse);
                        const float peb = two ? fast_exp2(sb - lse) : 0.0f;   // no second sample: no contribution
                        const float dsa = pea * (da - delta), dsb = peb * (db - delta);
                        const float2 dsa2 = make_float2(dsa, dsa), dsb2 = make_float2(dsb, dsb);
#pragma unroll
                        for (int e = 0; e < HP; ++e) dq[j][e] = __ffma2_rn(dsb2, ktb[e], __ffma2_rn(dsa2, kta[e], dq[j][e]));
                        if (i == li) {
                            my_a = dsa * p.sm_scale;
                            my_p = pea;
                        }
                        if (two && i + 1 == li) {
                            my_a = dsb * p.sm_scale;
                            my_p = peb;
                        }
                    }
                    for (int i = 0; !PAIRS && i < cnt; ++i) {
                        const uint32_t r = rec_slot<G, NG>(i, g) * 16u;
                        const uint4 wr = lds128(rec_w + r), pr = lds128(rec_p + r);
                        float w[4];
                        int pix[4] = { (int)pr.x, (int)pr.y, (int)pr.z, (int)pr.w };
                        // DCOORDS: 1-D weights and the inside flags (see publish_record_dc)
                        float wx0 = 0.0f, wx1 = 0.0f, wy0 = 0.0f, wy1 = 0.0f;
                        uint32_t flags = 0;
                        if constexpr (DCOORDS) {
                            wx0 = __uint_as_float(wr.x); wx1 = __uint_as_float(wr.y);
                            wy0 = __uint_as_float(wr.z); wy1 = __uint_as_float(wr.w);
                            w[0] = wx0 * wy0; w[1] = wx1 * wy0; w[2] = wx0 * wy1; w[3] = wx1 * wy1;
                            flags = pr.x >> 28;
                            pix[0] = (int)(pr.x & kPixMask);
                        } else {
                            w[0] = __uint_as_float(wr.x); w[1] = __uint_as_float(wr.y);
                            w[2] = __uint_as_float(wr.z); w[3] = __uint_as_float(wr.w);
                        }
                        const float2 w2[4] = { make_float2(w[0], w[0]), make_float2(w[1], w[1]),
                                               make_float2(w[2], w[2]), make_float2(w[3], w[3]) };
                        float2 kt[HP];
                        float sc, dp;        // logit in base-2 units, dout.v~
                        float ax = 0.0f, ay = 0.0f, bx = 0.0f, by = 0.0f;  // DCOORDS: d/dx, d/dy of q.k~ and dout.v~
                        if constexpr (!DCOORDS) {
                            float2 vt[HP];
                            gather_interp<T, D, STAGED>(kmap, pix, w2, li, kt);
                            gather_interp<T, D, STAGED>(vmap, pix, w2, li, vt);
                            float2 ps = __fmul2_rn(qf[0], kt[0]), pd = __fmul2_rn(dof[0], vt[0]);
#pragma unroll
                            for (int e = 1; e < HP; ++e) {
                                ps = __ffma2_rn(qf[e], kt[e], ps);
                                pd = __ffma2_rn(dof[e], vt[e], pd);
                            }
                            sc = group_sum<G>(ps.x + ps.y);
                            dp = group_sum<G>(pd.x + pd.y);
                        } else {
                            // per-corner dots A_c = qf.K_c (qf carries scale2) and B_c = dout.V_c, as this
                            // lane's parts: what is needed of them (logit, dout.v~ and their derivatives
                            // along x and y) is linear in the dots with coefficients the whole group
                            // shares, so the six combinations are formed per lane and then summed over
                            // the group (six reductions instead of eight)
                            float2 ac[4];
                            corner_dots<T, D, STAGED, true>(kmap, pix, w2, li, qf, kt, ac);
                            float a4[4], b4[4];
#pragma unroll
                            for (int c = 0; c < 4; ++c) a4[c] = ac[c].x + ac[c].y;
                            if constexpr (sizeof(T) == 2) {
                                corner_dots16<T, D, STAGED>(vmap, pix, li, doraw, b4);
                            } else {
                                float2 bc[4], unused[HP];
                                corner_dots<T, D, STAGED, false>(vmap, pix, w2, li, dof, unused, bc);
#pragma unroll
                                for (int c = 0; c < 4; ++c) b4[c] = bc[c].x + bc[c].y;
                            }
                            // a corner outside the map has value zero: drop its dot
                            const float vx0 = (flags & 1u) ? 1.0f : 0.0f, vx1 = (flags & 2u) ? 1.0f : 0.0f;
                            const float vy0 = (flags & 4u) ? 1.0f : 0.0f, vy1 = (flags & 8u) ? 1.0f : 0.0f;
                            sc = group_sum<G>(w[0] * a4[0] + w[1] * a4[1] + w[2] * a4[2] + w[3] * a4[3]);
                            dp = group_sum<G>(w[0] * b4[0] + w[1] * b4[1] + w[2] * b4[2] + w[3] * b4[3]);
                            ax = group_sum<G>(wy0 * (vx1 * a4[1] - vx0 * a4[0]) + wy1 * (vx1 * a4[3] - vx0 * a4[2]));
                            ay = group_sum<G>(wx0 * (vy1 * a4[2] - vy0 * a4[0]) + wx1 * (vy1 * a4[3] - vy0 * a4[1]));
                            bx = group_sum<G>(wy0 * (vx1 * b4[1] - vx0 * b4[0]) + wy1 * (vx1 * b4[3] - vx0 * b4[2]));
                            by = group_sum<G>(wx0 * (vy1 * b4[2] - vy0 * b4[0]) + wx1 * (vy1 * b4[3] - vy0 * b4[1]));
                        }
                        const float pe = fast_exp2(sc - lse);
                        const float ds = pe * (dp - delta);
                        const float2 ds2 = make_float2(ds, ds);
#pragma unroll
                        for (int e = 0; e < HP; ++e) dq[j][e] = __ffma2_rn(ds2, kt[e], dq[j][e]);
                        if constexpr (DCOORDS) {
                            // sm_scale*ds*(q.dK_c/dx) = (ds*ln2)*ax because qf carries sm_scale*log2(e)
                            if (i == li) {
                                my_gx = ((ds * kLn2) * ax + pe * bx) * (float)(p.W - 1);
                                my_gy = ((ds * kLn2) * ay + pe * by) * (float)(p.H - 1);
                            }
                        }
                        if constexpr (TWOPASS) {
                            if (i == li) {
                                my_a = ds * p.sm_scale;
                                my_p = pe;
                            }
                        }
                        // qf carries scale2 = sm_scale*log2(e): sm_scale*ds*q = (ds*ln2)*qf
                        const float ck = ds * kLn2;
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            if constexpr (TWOPASS) continue;
                            if (!live || w[c] == 0.0f) continue;
                            const float wk = ck * w[c], wv = pe * w[c];
#pragma unroll
                            for (int ch = 0; ch < CH; ++ch) {
                                const int h0 = ch * HV;
                                const size_t off = (size_t)pix[c] * D + (size_t)(ch * G + li) * EPV;
                                if constexpr (PRIV) {
                                    const uint32_t ak = acc_k + (uint32_t)off * 4u, av = acc_v + (uint32_t)off * 4u;
#pragma unroll
                                    for (int e = 0; e < HV; ++e) {
                                        red_shared_add(ak + 8u * e, wk * qf[h0 + e].x);
                                        red_shared_add(ak + 8u * e + 4u, wk * qf[h0 + e].y);
                                        red_shared_add(av + 8u * e, wv * dof[h0 + e].x);
                                        red_shared_add(av + 8u * e + 4u, wv * dof[h0 + e].y);
                                    }
                                } else {
#pragma unroll
                                    for (int e = 0; e < HV; e += 2) {
                                        red_global_add_v4(dkmap + off + 2 * e, wk * qf[h0 + e].x, wk * qf[h0 + e].y,
                                                          wk * qf[h0 + e + 1].x, wk * qf[h0 + e + 1].y);
                                        red_global_add_v4(dvmap + off + 2 * e, wv * dof[h0 + e].x, wv * dof[h0 + e].y,
                                                          wv * dof[h0 + e + 1].x, wv * dof[h0 + e + 1].y);
                                    }
                                }
                            }
                        }
                    }
                    if constexpr (TWOPASS) {
                        // one coalesced float2 per lane: the group writes G samples at once
                        if (live && li < cnt) scal_row[s0 + li] = make_float2(my_a, my_p);
                    }
                    if constexpr (DCOORDS) {
                        // all heads add into the same coordinate gradient
                        if (live && li < cnt) {
                            float* dst = p.dcoords + (((((size_t)b * p.V + vq) * p.L + l) * p.V + vk) * (size_t)p.S + s0 + li) * 2;
                            asm volatile("red.global.add.v2.f32 [%0], {%1,%2};" :: "l"(dst), "f"(my_gx), "f"(my_gy) : "memory");
                        }
                    }
                    __syncwarp();
                }
            }
        }
        if constexpr (STAGED) {
            if (__syncthreads_or(ok ? 0 : 1)) return;
            if (p.nstage == 1 && vk + 1 < p.V && threadIdx.x == 0) {
                stage_maps(smem0, kmaps + (size_t)(vk + 1) * map_stride_view, vmaps + (size_t)(vk + 1) * map_stride_view,
                           p.map_bytes, bar0);
            }
            if constexpr (PRIV) {
                // flush this key view's private dK/dV maps with vector reductions and clear them
                const uint32_t nvec = p.acc_bytes / 16u;
                for (uint32_t i = threadIdx.x; i < 2u * nvec; i += blockDim.x) {
                    const uint32_t sa = acc_k + i * 16u;
                    const uint4 r = lds128(sa);
                    if ((r.x | r.y | r.z | r.w) == 0u) continue;
                    float* dst = (i < nvec ? dkmap + (size_t)i * 4 : dvmap + (size_t)(i - nvec) * 4);
                    red_global_add_v4(dst, __uint_as_float(r.x), __uint_as_float(r.y), __uint_as_float(r.z),
                                      __uint_as_float(r.w));
                    sts128(sa, make_uint4(0, 0, 0, 0));
                }
                __syncthreads();
            }
        }
    }

#pragma unroll
    for (int j = 0; j < NQ; ++j) {
        const int qi = q0 + j * slot_stride + warp * NG + g;
        if (qi >= qend) continue;
        const int vq = qi / p.L, l = qi - vq * p.L;
        const size_t qrow = (((size_t)b * p.V + vq) * p.Hh + h) * p.L + l;
#pragma unroll
        for (int ch = 0; ch < CH; ++ch) {
            float f[EPV];
#pragma unroll
            for (int e = 0; e < HV; ++e) {
                f[2 * e] = dq[j][ch * HV + e].x * p.sm_scale;
                f[2 * e + 1] = dq[j][ch * HV + e].y * p.sm_scale;
            }
            const uint4 packed = pack16(f, (T*)nullptr);
            stg128((char*)p.dq + qrow * ROWB + (size_t)(ch * G + li) * 16, packed);
            if (p.dq_mirror) stg128((char*)p.dq_mirror + qrow * ROWB + (size_t)(ch * G + li) * 16, packed);
        }
    }
}

// fp32 accumulators -> storage type, 8 elements per thread.
template <typename T>
__global__ void cast_from_f32_kernel(const float* __restrict__ src, T* __restrict__ dst, size_t n8) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
        const uint4 a = ldg128_stream(src + i * 8), c = ldg128_stream(src + i * 8 + 4);
        const float f[8] = { __uint_as_float(a.x), __uint_as_float(a.y), __uint_as_float(a.z), __uint_as_float(a.w),
                             __uint_as_float(c.x), __uint_as_float(c.y), __uint_as_float(c.z), __uint_as_float(c.w) };
        stg128(dst + i * 8, pack16(f, (T*)nullptr));
    }
}

}  // namespace dsdpa

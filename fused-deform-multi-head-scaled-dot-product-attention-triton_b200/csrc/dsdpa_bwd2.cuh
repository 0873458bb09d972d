// Backward, two-pass form: dK/dV as a GATHER over pixel-sorted sample lists.
//
// The reference scatters every sample's contribution into dK/dV with scalar fp32
// atomics (ops/triton.py:342-360; "TODO: reduce atomic conflict", ops/triton.py:341).
// Here the same sums are formed without any atomic and in a fixed order:
//
//   1. index_build_kernel   (per batch element, gather tile and key view; shared by all
//      heads, since coordinates are, ops/torch.py:10): a counting sort of the tile's
//      (sample, corner) pairs by key pixel.  Output per segment: row pointers [L+1] and
//      entries {query-in-tile | sample<<16, weight}, each pixel's entries in a fixed
//      canonical order.
//   2. bwd_scatter_kernel<..., TWOPASS>  (dsdpa_bwd.cuh): recomputes p and ds per sample,
//      writes dq and the per-sample scalars (sm_scale*ds, p).
//   3. bwd_gather_kernel    (per batch element, head and key view): for every gather tile
//      loads the tile's q rows, dout rows and scalars into shared memory, then each group
//      of lanes walks the entry list of one key pixel at a time, accumulating
//          dK[pix] += (sm_scale*ds * w) * q[query],   dV[pix] += (p * w) * dout[query]
//      in registers, and adds the result to the fp32 dK/dV maps in global memory, which
//      this CTA alone owns (plain read-modify-write, tiles in order).
//
// A gather tile is a run of QB consecutive pixels of one query view (tpv tiles per view).
#pragma once

#include "dsdpa_common.cuh"

namespace dsdpa {

struct IndexParams {
    const float* coords;
    int* rowptr;      // [B*T*V segments][L+1]
    uint2* entries;   // [B*T*V segments][QB*S*4]
    int B, V, W, H, L, S;
    float hw, hh;
    int tpv, QB;      // T = V*tpv tiles per batch element
};

constexpr int kIndexWarpsDefault = 8;

// Shared memory: cnt[NWARPS][L] ints, then part[NWARPS*32] ints.  (A template so that
// the header can be included by several translation units.)
template <int NWARPS>
__global__ void __launch_bounds__(NWARPS * 32) index_build_kernel(const IndexParams p) {
    static_assert(NWARPS == 8, "the scan below handles 256 partial sums");
    constexpr int kIndexWarps = NWARPS;
    extern __shared__ __align__(16) unsigned char smem[];
    int* cnt = reinterpret_cast<int*>(smem);
    int* part = cnt + kIndexWarps * p.L;

    const int T = p.V * p.tpv;
    const int seg = blockIdx.x;
    const int vk = seg % p.V;
    const int t = (seg / p.V) % T;
    const int b = seg / (p.V * T);
    const int vq = t / p.tpv, tl = t - vq * p.tpv;
    const int l0 = tl * p.QB;
    const int len = min(p.QB, p.L - l0);
    const int nsamp = len * p.S;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // each warp owns a contiguous run of samples (a multiple of 32 of them)
    const int per_warp = ((nsamp + kIndexWarps * 32 - 1) / (kIndexWarps * 32)) * 32;
    const int wbeg = warp * per_warp, wend = min(wbeg + per_warp, nsamp);
    int* mycnt = cnt + warp * p.L;

    for (int i = threadIdx.x; i < kIndexWarps * p.L; i += blockDim.x) cnt[i] = 0;
    __syncthreads();

    // sample index (within the tile) -> coordinates; samples are ordered (query, s)
    auto coord_of = [&](int smp) -> float2 {
        const int ql = smp / p.S, s = smp - ql * p.S;
        const size_t row = ((((size_t)b * p.V + vq) * p.L + (l0 + ql)) * p.V + vk) * (size_t)p.S + s;
        return __ldg(reinterpret_cast<const float2*>(p.coords) + row);
    };

    // pass 1: per-warp histogram of key pixels
    for (int base = wbeg; base < wend; base += 32) {
        const int smp = base + lane;
        if (smp < wend) {
            const float2 c = coord_of(smp);
            Corners cr;
            float fx, fy;
            decode_corners(c.x, c.y, p.W, p.H, p.hw, p.hh, cr, fx, fy);
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (cr.w[k] != 0.0f) atomicAdd(&mycnt[cr.pix[k]], 1);
        }
    }
    __syncthreads();

    // pass 2: exclusive scan over pixels of the per-pixel totals -> row pointers, and
    // per-warp start offsets inside each pixel's list (warp order = canonical order)
    const int nthr = blockDim.x;
    const int chunk = (p.L + nthr - 1) / nthr;
    const int pbeg = min((int)threadIdx.x * chunk, p.L), pend = min(pbeg + chunk, p.L);
    int local = 0;
    for (int pix = pbeg; pix < pend; ++pix)
        for (int w = 0; w < kIndexWarps; ++w) local += cnt[w * p.L + pix];
    part[threadIdx.x] = local;
    __syncthreads();
    if (warp == 0) {
        // scan of 256 partial sums by one warp, 8 per lane
        int v[8], sum = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) { v[i] = part[lane * 8 + i]; sum += v[i]; }
        int incl = sum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += n;
        }
        int run = incl - sum;
#pragma unroll
        for (int i = 0; i < 8; ++i) { part[lane * 8 + i] = run; run += v[i]; }
    }
    __syncthreads();
    int* rowptr = p.rowptr + (size_t)seg * (p.L + 1);
    int run = part[threadIdx.x];
    for (int pix = pbeg; pix < pend; ++pix) {
        rowptr[pix] = run;
        for (int w = 0; w < kIndexWarps; ++w) {
            const int c = cnt[w * p.L + pix];
            cnt[w * p.L + pix] = run;
            run += c;
        }
    }
    if (pend == p.L && pbeg < p.L) rowptr[p.L] = run;
    if (p.L == 0 && threadIdx.x == 0) rowptr[0] = 0;
    __syncthreads();

    // pass 3: scatter in canonical order (32 samples at a time, corner-major inside),
    // ranks of equal pixels inside the warp from match_any
    uint2* entries = p.entries + (size_t)seg * ((size_t)p.QB * p.S * 4);
    for (int base = wbeg; base < wend; base += 32) {
        const int smp = base + lane;
        Corners cr;
        cr.w[0] = cr.w[1] = cr.w[2] = cr.w[3] = 0.0f;
        cr.pix[0] = cr.pix[1] = cr.pix[2] = cr.pix[3] = 0;
        unsigned tag = 0;
        if (smp < wend) {
            const float2 c = coord_of(smp);
            float fx, fy;
            decode_corners(c.x, c.y, p.W, p.H, p.hw, p.hh, cr, fx, fy);
            const int ql = smp / p.S, s = smp - ql * p.S;
            tag = (unsigned)ql | ((unsigned)s << 16);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const bool valid = cr.w[k] != 0.0f;
            const unsigned vmask = __ballot_sync(0xffffffffu, valid);
            if (valid) {
                const int pix = cr.pix[k];
                const unsigned same = __match_any_sync(vmask, pix);
                const int leader = __ffs(same) - 1;
                const int rank = __popc(same & ((1u << lane) - 1u));
                int start = 0;
                if (lane == leader) {
                    start = mycnt[pix];
                    mycnt[pix] = start + __popc(same);
                }
                start = __shfl_sync(same, start, leader);
                entries[start + rank] = make_uint2(tag, __float_as_uint(cr.w[k]));
            }
            __syncwarp();
        }
    }
}

struct GatherParams {
    const void* q;
    const void* dout;
    const float2* scal;
    const int* rowptr;
    const uint2* entries;
    float* dk32;
    float* dv32;
    int B, V, Hh, L, S;
    int tpv, QB;
    int* err;
};

template <typename T, int D>
__global__ void __launch_bounds__(512, 1) bwd_gather_kernel(const GatherParams p) {
    using RC = RowCfg<T, D>;
    constexpr int G = RC::G, NG = RC::NG, EPL = RC::EPL, CH = RC::CH, EPV = RC::EPV, ROWB = RC::ROWB;
    extern __shared__ __align__(128) unsigned char smem[];

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int g = lane / G, li = lane % G;
    const int ngroups = nw * NG, gid = warp * NG + g;
    // heads of one (batch, key view) are neighbours in the grid: they share the index
    const int h = blockIdx.x % p.Hh;
    const int vk = (blockIdx.x / p.Hh) % p.V;
    const int b = blockIdx.x / (p.Hh * p.V);
    const int NT = p.V * p.tpv;  // gather tiles per batch element

    const uint32_t smem0 = smem_addr(smem);
    const uint32_t q_s = smem0;
    const uint32_t do_s = q_s + (uint32_t)p.QB * ROWB;
    const uint32_t sc_s = do_s + (uint32_t)p.QB * ROWB;
    const uint32_t bar = sc_s + (((uint32_t)p.QB * p.S * 8u + 15u) & ~15u);

    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
        fence_proxy_async();
    }
    __syncthreads();

    float* dkmap = p.dk32 + (((size_t)b * p.V + vk) * p.Hh + h) * (size_t)p.L * D;
    float* dvmap = p.dv32 + (((size_t)b * p.V + vk) * p.Hh + h) * (size_t)p.L * D;

    for (int t = 0; t < NT; ++t) {
        const int vq = t / p.tpv, tl = t - vq * p.tpv;
        const int l0 = tl * p.QB;
        const int len = min(p.QB, p.L - l0);
        if (threadIdx.x == 0) {
            const size_t qrow0 = (((size_t)b * p.V + vq) * p.Hh + h) * p.L + l0;
            const size_t tile = ((size_t)b * p.Hh + h) * (size_t)NT + t;
            const float2* sc = p.scal + ((tile * p.V + vk) * (size_t)p.QB) * (size_t)p.S;
            // a bulk copy moves multiples of 16 bytes: an odd count of 8-byte scalars is rounded
            // up (the source buffer is padded, the shared-memory slot is sized for it)
            const unsigned rows_b = (unsigned)len * ROWB, sc_b = ((unsigned)len * p.S * 8u + 15u) & ~15u;
            fence_proxy_async();
            mbar_expect_tx(bar, 2u * rows_b + sc_b);
            bulk_g2s_chunked(q_s, (const char*)p.q + qrow0 * ROWB, rows_b, bar);
            bulk_g2s_chunked(do_s, (const char*)p.dout + qrow0 * ROWB, rows_b, bar);
            bulk_g2s_chunked(sc_s, (const char*)sc, sc_b, bar);
        }
        bool ok = mbar_wait_bounded(bar, (unsigned)t & 1u, p.err);
        ok = __all_sync(0xffffffffu, ok);

        if (ok) {
            const size_t seg = ((size_t)b * NT + t) * p.V + vk;
            const int* rowptr = p.rowptr + seg * (p.L + 1);
            const uint2* entries = p.entries + seg * ((size_t)p.QB * p.S * 4);
            for (int pix = gid; pix < p.L; pix += ngroups) {
                const int beg = __ldg(rowptr + pix), end = __ldg(rowptr + pix + 1);
                if (beg == end) continue;
                float ak[EPL], av[EPL];
#pragma unroll
                for (int e = 0; e < EPL; ++e) ak[e] = av[e] = 0.0f;
                for (int e0 = beg; e0 < end; e0 += 4) {
                    // four entries in flight; a clamped repeat of the last one gets weight 0
                    uint2 ent[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) ent[u] = __ldg(entries + min(e0 + u, end - 1));
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const uint32_t ql = ent[u].x & 0xffffu, s = ent[u].x >> 16;
                        const float w = e0 + u < end ? __uint_as_float(ent[u].y) : 0.0f;
                        float2 sc;
                        asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];"
                                     : "=f"(sc.x), "=f"(sc.y) : "r"(sc_s + (ql * (uint32_t)p.S + s) * 8u));
                        const float aw = sc.x * w, pw = sc.y * w;
#pragma unroll
                        for (int ch = 0; ch < CH; ++ch) {
                            float fq[EPV], fd[EPV];
                            unpack16(lds128(q_s + ql * ROWB + (uint32_t)(ch * G + li) * 16u), fq, (T*)nullptr);
                            unpack16(lds128(do_s + ql * ROWB + (uint32_t)(ch * G + li) * 16u), fd, (T*)nullptr);
#pragma unroll
                            for (int k = 0; k < EPV; ++k) {
                                ak[ch * EPV + k] = fmaf(aw, fq[k], ak[ch * EPV + k]);
                                av[ch * EPV + k] = fmaf(pw, fd[k], av[ch * EPV + k]);
                            }
                        }
                    }
                }
                // this CTA alone owns the (batch, head, key view) maps: plain read-modify-write
#pragma unroll
                for (int ch = 0; ch < CH; ++ch)
#pragma unroll
                    for (int k = 0; k < EPV; k += 4) {
                        const size_t off = (size_t)pix * D + (size_t)(ch * G + li) * EPV + k;
                        float4* pk = reinterpret_cast<float4*>(dkmap + off);
                        float4* pv = reinterpret_cast<float4*>(dvmap + off);
                        float4 a = *pk, c = *pv;
                        a.x += ak[ch * EPV + k]; a.y += ak[ch * EPV + k + 1];
                        a.z += ak[ch * EPV + k + 2]; a.w += ak[ch * EPV + k + 3];
                        c.x += av[ch * EPV + k]; c.y += av[ch * EPV + k + 1];
                        c.z += av[ch * EPV + k + 2]; c.w += av[ch * EPV + k + 3];
                        *pk = a;
                        *pv = c;
                    }
            }
        }
        // every group is done with the tile (and its global updates are ordered before the
        // next tile's by the barrier) before the buffers are refilled
        if (__syncthreads_or(ok ? 0 : 1)) return;
    }
}

}  // namespace dsdpa

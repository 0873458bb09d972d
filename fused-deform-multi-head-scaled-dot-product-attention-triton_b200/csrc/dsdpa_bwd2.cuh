// Backward, two-pass form: dK/dV as a GATHER over pixel-sorted sample lists.
//
// The reference scatters every sample's contribution into dK/dV with scalar fp32
// atomics (ops/triton.py:342-360; "TODO: reduce atomic conflict", ops/triton.py:341).
// Here the same sums are formed without any atomic and in a fixed order:
//
//   1. index_build_kernel   (per batch element, gather tile and key view; shared by all
//      heads, since coordinates are, ops/torch.py:10): a counting sort of the tile's
//      (sample, corner) pairs by key pixel.  Output per segment: row pointers [L+1] and
//      entries {row offset of the query in the tile | index of the sample's scalars << 16,
//      weight}, each pixel's entries in a fixed canonical order and padded with zero-weight
//      entries to a multiple of four (the gather pass reads four entries per step).
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
    int rowb16;       // bytes of one q row in the gather tile / 16
    int seg_entries;  // entries reserved per segment (QB*S*4 + 3*L, rounded up to 4)
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
    for (int pix = pbeg; pix < pend; ++pix) {
        int tot = 0;
        for (int w = 0; w < kIndexWarps; ++w) tot += cnt[w * p.L + pix];
        local += (tot + 3) & ~3;  // every list is padded to a multiple of four entries
    }
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
        int at = run;
        for (int w = 0; w < kIndexWarps; ++w) {
            const int c = cnt[w * p.L + pix];
            cnt[w * p.L + pix] = at;
            at += c;
        }
        run += (at - run + 3) & ~3;
    }
    if (pend == p.L && pbeg < p.L) rowptr[p.L] = run;
    if (p.L == 0 && threadIdx.x == 0) rowptr[0] = 0;
    __syncthreads();

    // pass 3: scatter in canonical order (32 samples at a time, corner-major inside),
    // ranks of equal pixels inside the warp from match_any
    uint2* entries = p.entries + (size_t)seg * (size_t)p.seg_entries;
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
            const int ql = smp / p.S;
            // what the gather pass needs of the sample: where its query's row starts in the tile
            // (in 16-byte units) and which of the tile's scalar pairs is its own
            tag = (unsigned)(ql * p.rowb16) | ((unsigned)smp << 16);
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
    __syncthreads();
    // zero-weight padding behind every list (the last warp's cursor marks the list's end)
    for (int pix = pbeg; pix < pend; ++pix) {
        int at = cnt[(kIndexWarps - 1) * p.L + pix];
        const int padded = (at + 3) & ~3;
        for (; at < padded; ++at) entries[at] = make_uint2(0u, 0u);
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
    // where the finished maps go: dk/dv in the storage type (equal to dk32/dv32 for fp32 storage,
    // which accumulates in place) and the optional mirrors (may be another GPU's memory)
    void* dk;
    void* dv;
    void* dk_mirror;
    void* dv_mirror;
    int B, V, Hh, L, S;
    int tpv, QB;
    int seg_entries;
    int nslab;            // CTAs per (batch, head, key view)
    int* err;
};

// After the last tile: a group owns the same key pixels in every tile, and each lane the same
// elements of their rows, so it hands its finished rows over itself (reading back what it wrote,
// or the zero fill): rounded to the storage type into dK/dV, and into the mirrors.  These stores
// are spread over the time the CTAs of the grid finish at.  (Everything it needs is derived
// again from the block and thread index, so that nothing stays live across the tile loop for it.)
template <typename T, int D>
__device__ __forceinline__ void gather_hand_over(const GatherParams& p) {
    using RC = RowCfg<T, D>;
    constexpr int G = RC::G, NG = RC::NG, CH = RC::CH, EPV = RC::EPV, ROWB = RC::ROWB;
    const bool narrow = sizeof(T) == 2;
    if (!narrow && !p.dk_mirror && !p.dv_mirror) return;
    // (read through volatile asm: the compiler then derives these values anew instead of
    // carrying the tile loop's copies in registers through that loop)
    unsigned tid, cta, ntid;
    asm volatile("mov.u32 %0, %%tid.x;" : "=r"(tid));
    asm volatile("mov.u32 %0, %%ctaid.x;" : "=r"(cta));
    asm volatile("mov.u32 %0, %%ntid.x;" : "=r"(ntid));
    const int lane = tid & 31, warp = tid >> 5, nw = ntid >> 5;
    const int g = lane / G, li = lane % G;
    const int slab = cta % p.nslab, unit = cta / p.nslab;
    const int ngroups = nw * NG * p.nslab, gid = (warp * NG + g) * p.nslab + slab;
    const size_t map = (size_t)unit / p.Hh % p.V + (size_t)p.V * (unit / (p.Hh * p.V));  // b*V + vk
    const size_t map_row0 = (map * p.Hh + unit % p.Hh) * (size_t)p.L;
    // one map after the other (K, then V) keeps the loop's register need small
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {
        const float* acc = (which ? p.dv32 : p.dk32) + map_row0 * D;
        void* dst = which ? p.dv : p.dk;
        void* mir = which ? p.dv_mirror : p.dk_mirror;
        char* o_loc = narrow ? (char*)dst + map_row0 * ROWB : nullptr;
        char* o_mir = mir ? (char*)mir + map_row0 * ROWB : nullptr;
        if (!o_loc && !o_mir) continue;
#pragma unroll 2
        for (int pix = gid; pix < p.L; pix += ngroups) {
#pragma unroll
            for (int ch = 0; ch < CH; ++ch) {
                float f[EPV];
#pragma unroll
                for (int k = 0; k < EPV / 4; ++k) {
                    const float4 a = *reinterpret_cast<const float4*>(acc + (size_t)pix * D + (size_t)(ch * G + li) * EPV + 4 * k);
                    f[4 * k] = a.x; f[4 * k + 1] = a.y; f[4 * k + 2] = a.z; f[4 * k + 3] = a.w;
                }
                const uint4 packed = pack16(f, (T*)nullptr);
                const size_t o = (size_t)pix * ROWB + (size_t)(ch * G + li) * 16;
                if (o_loc) stg128(o_loc + o, packed);
                if (o_mir) stg128(o_mir + o, packed);
            }
        }
    }
}

// Shared memory of one tile: q rows and dout rows in the storage type ([QB, D] each), then
// the tile's scalars ([QB, S] float2), then the mbarrier; all three filled by bulk copies.
template <typename T, int D>
__global__ void __launch_bounds__(768, 1) bwd_gather_kernel(const GatherParams p) {
    using RC = RowCfg<T, D>;
    constexpr int G = RC::G, NG = RC::NG, CH = RC::CH, EPV = RC::EPV, ROWB = RC::ROWB;
    constexpr int HV = EPV / 2, HP = RC::EPL / 2;
    extern __shared__ __align__(128) unsigned char smem[];

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int g = lane / G, li = lane % G;
    // (nslab > 1: several CTAs share one (batch, head, key view) and split its key pixels, which
    // evens out the last wave of a small grid; each still loads every tile)
    const int slab = blockIdx.x % p.nslab, unit = blockIdx.x / p.nslab;
    // groups of all CTAs that share the maps, and this group's rank among them
    const int ngroups = nw * NG * p.nslab, gid = (warp * NG + g) * p.nslab + slab;
    // heads of one (batch, key view) are neighbours in the grid: they share the index
    const int h = unit % p.Hh;
    const int vk = (unit / p.Hh) % p.V;
    const int b = unit / (p.Hh * p.V);
    const int NT = p.V * p.tpv;  // gather tiles per batch element

    const uint32_t smem0 = smem_addr(smem);
    const uint32_t q_s = smem0 + (uint32_t)li * 16u;             // this lane's slice of row 0
    const uint32_t do_s = q_s + (uint32_t)p.QB * ROWB;
    const uint32_t sc_s = smem0 + 2u * (uint32_t)p.QB * ROWB;
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
            bulk_g2s_chunked(smem0, (const char*)p.q + qrow0 * ROWB, rows_b, bar);
            bulk_g2s_chunked(smem0 + (uint32_t)p.QB * ROWB, (const char*)p.dout + qrow0 * ROWB, rows_b, bar);
            bulk_g2s_chunked(sc_s, (const char*)sc, sc_b, bar);
        }
        bool ok = mbar_wait_bounded(bar, (unsigned)t & 1u, p.err);
        ok = __all_sync(0xffffffffu, ok);

        if (ok) {
            const size_t seg = ((size_t)b * NT + t) * p.V + vk;
            const int* rowptr = p.rowptr + seg * (p.L + 1);
            const uint4* entries4 = reinterpret_cast<const uint4*>(p.entries + seg * (size_t)p.seg_entries);
            // Key pixels are dealt round-robin to the groups: neighbouring pixels have lists of
            // similar length (also when the coordinates cluster), so the groups stay balanced.
            // The walk is software-pipelined: the row pointers of the pixel after next and the
            // first entries of the next pixel are requested before the current pixel's entries
            // are processed, so that their L2 latency hides behind that work.
            int pix = gid;
            int beg = 0, end = 0, nbeg = 0, nend = 0;
            if (pix < p.L) { beg = __ldg(rowptr + pix); end = __ldg(rowptr + pix + 1); }
            if (pix + ngroups < p.L) { nbeg = __ldg(rowptr + pix + ngroups); nend = __ldg(rowptr + pix + ngroups + 1); }
            uint4 first0 = make_uint4(0, 0, 0, 0), first1 = first0;
            if (end > beg) { first0 = __ldg(entries4 + (beg >> 1)); first1 = __ldg(entries4 + (beg >> 1) + 1); }
            while (pix < p.L) {
                int n2beg = 0, n2end = 0;
                if (pix + 2 * ngroups < p.L) {
                    n2beg = __ldg(rowptr + pix + 2 * ngroups);
                    n2end = __ldg(rowptr + pix + 2 * ngroups + 1);
                }
                uint4 nfirst0 = make_uint4(0, 0, 0, 0), nfirst1 = nfirst0;
                if (nend > nbeg) { nfirst0 = __ldg(entries4 + (nbeg >> 1)); nfirst1 = __ldg(entries4 + (nbeg >> 1) + 1); }
                if (end > beg) {
                    // this CTA alone owns the (batch, head, key view) maps, so the update is a plain
                    // read-modify-write; the read is issued now and hides behind the entry loop
                    float4 gk[CH * (EPV / 4)], gv[CH * (EPV / 4)];
#pragma unroll
                    for (int ch = 0; ch < CH; ++ch)
#pragma unroll
                        for (int k = 0; k < EPV / 4; ++k) {
                            const size_t off = (size_t)pix * D + (size_t)(ch * G + li) * EPV + 4 * k;
                            gk[ch * (EPV / 4) + k] = *reinterpret_cast<const float4*>(dkmap + off);
                            gv[ch * (EPV / 4) + k] = *reinterpret_cast<const float4*>(dvmap + off);
                        }
                    float2 ak[HP], av[HP];
#pragma unroll
                    for (int e = 0; e < HP; ++e) ak[e] = av[e] = make_float2(0.0f, 0.0f);
                    // four entries (32 bytes) per step, the next four already in flight; lists are
                    // padded to a multiple of four with zero-weight entries
                    uint4 nx0 = first0, nx1 = first1;
                    for (int e0 = beg; e0 < end; e0 += 4) {
                        const uint4 c0 = nx0, c1 = nx1;
                        if (e0 + 4 < end) {
                            nx0 = __ldg(entries4 + ((e0 + 4) >> 1));
                            nx1 = __ldg(entries4 + ((e0 + 4) >> 1) + 1);
                        }
                        const uint32_t tags[4] = { c0.x, c0.z, c1.x, c1.z };
                        const float ws[4] = { __uint_as_float(c0.y), __uint_as_float(c0.w), __uint_as_float(c1.y),
                                              __uint_as_float(c1.w) };
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const uint32_t roff = (tags[u] & 0xffffu) << 4, soff = (tags[u] >> 16) << 3;
                            float2 sc;
                            asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(sc.x), "=f"(sc.y) : "r"(sc_s + soff));
                            const float aw = sc.x * ws[u], pw = sc.y * ws[u];
                            const float2 aw2 = make_float2(aw, aw), pw2 = make_float2(pw, pw);
#pragma unroll
                            for (int ch = 0; ch < CH; ++ch) {
                                float2 fq[HV], fd[HV];
                                unpack16_pairs(lds128(q_s + roff + (uint32_t)(ch * G) * 16u), fq, (T*)nullptr);
                                unpack16_pairs(lds128(do_s + roff + (uint32_t)(ch * G) * 16u), fd, (T*)nullptr);
#pragma unroll
                                for (int k = 0; k < HV; ++k) {
                                    ak[ch * HV + k] = __ffma2_rn(aw2, fq[k], ak[ch * HV + k]);
                                    av[ch * HV + k] = __ffma2_rn(pw2, fd[k], av[ch * HV + k]);
                                }
                            }
                        }
                    }
#pragma unroll
                    for (int ch = 0; ch < CH; ++ch)
#pragma unroll
                        for (int k = 0; k < EPV / 4; ++k) {
                            const size_t off = (size_t)pix * D + (size_t)(ch * G + li) * EPV + 4 * k;
                            float4 a = gk[ch * (EPV / 4) + k], c = gv[ch * (EPV / 4) + k];
                            const int e = ch * HV + 2 * k;
                            a.x += ak[e].x; a.y += ak[e].y; a.z += ak[e + 1].x; a.w += ak[e + 1].y;
                            c.x += av[e].x; c.y += av[e].y; c.z += av[e + 1].x; c.w += av[e + 1].y;
                            *reinterpret_cast<float4*>(dkmap + off) = a;
                            *reinterpret_cast<float4*>(dvmap + off) = c;
                        }
                }
                pix += ngroups;
                beg = nbeg; end = nend;
                nbeg = n2beg; nend = n2end;
                first0 = nfirst0; first1 = nfirst1;
            }
        }
        // every group is done with the tile before its buffers are refilled
        if (__syncthreads_or(ok ? 0 : 1)) return;
    }

    gather_hand_over<T, D>(p);
}

}  // namespace dsdpa

// Backward, two-pass form: dK/dV as a GATHER over sorted sample lists.
//
// The reference scatters every sample's contribution into dK/dV with scalar fp32
// atomics (ops/triton.py:342-360; "TODO: reduce atomic conflict", ops/triton.py:341).
// Here the same sums are formed without colliding atomics and in a fixed order:
//
//   1. index_build_kernel   (per batch element, gather tile and key view; shared by all
//      heads, since coordinates are, ops/torch.py:10): a counting sort of the tile's samples
//      by ANCHOR.  The two corners of a sample that lie in one map row, (x0, y) and (x0+1, y),
//      are neighbours in memory and receive the same query's rows, so they travel as one
//      entry: anchor (y, a) with a = x0+1 in [0, W] stands for the pixel pair (a-1, a) of row y
//      (a = 0 and a = W: one of the two lies outside the map and carries weight zero).  A sample
//      gives up to two entries, one per map row of its footprint.  Output per segment: 16-byte
//      entries {byte offset of the query's row in the tile, byte offset of the sample's scalars,
//      weight of the left pixel, weight of the right pixel}, each anchor's entries in a fixed
//      canonical order, and a work list of the non-empty anchors {right pixel, first entry, end,
//      column} sorted by list length, longest first (per slab of map rows when several CTAs
//      share a map): lanes that work side by side then get lists of equal length, and dealing
//      the sorted list out back and forth gives every group the same amount of work.
//   2. bwd_scatter_kernel<..., TWOPASS>  (dsdpa_bwd.cuh): recomputes p and ds per sample,
//      writes dq and the per-sample scalars (sm_scale*ds, p).
//   3. bwd_gather_kernel    (per batch element, head and key view): for every gather tile
//      loads the tile's q rows, dout rows and scalars into shared memory, then each group
//      of lanes walks the entry list of one anchor at a time, accumulating for both pixels
//          dK[pix] += (sm_scale*ds * w) * q[query],   dV[pix] += (p * w) * dout[query]
//      in registers -- one read of the query's rows serves both -- and adds the sums to fp32
//      maps in global memory.  A pixel is the left one of one anchor and the right one of the
//      next, so there are two sets of maps, "left" and "right": every map element then has
//      exactly one writer (the same lanes in every tile, in tile order), no two additions ever
//      race, and the result is reproducible bit for bit.  After the last tile the CTA adds the
//      two sets and hands the finished rows over (storage type, mirrors).
//
// A gather tile is a run of QB consecutive pixels of one query view (tpv tiles per view).
#pragma once

#include "dsdpa_common.cuh"
#include "dsdpa_plan.h"

namespace dsdpa {

struct IndexParams {
    const float* coords;
    int4* sched;      // [B*T*V segments][A] work list: {right pixel, first entry, end, anchor column}
    int2* sched_hdr;  // [B*T*V segments][nslab] {first record of the slab, non-empty anchors in it}
    uint4* entries;   // [B*T*V segments][seg_entries]
    int B, V, W, H, L, S;
    float hw, hh;
    int tpv, QB;      // T = V*tpv tiles per batch element
    int rowb;         // bytes of one q row in the gather tile
    int seg_entries;  // entries reserved per segment (2*QB*S)
    int A;            // anchors per map: H*(W+1)
    int nhist;        // warps that take samples, each with a histogram of its own (1..NWARPS)
    int nslab;        // slabs of map rows the gather pass splits a map into (1..kMaxSlabs)
    int* err;         // device error word
};

constexpr int kMaxSlabs = 4;
constexpr int kLenBuckets = 512;   // list lengths are sorted exactly up to this, longer ones count as equal

constexpr int kIndexWarpsDefault = 16;   // the build is bound by latency: as many warps as the histograms allow

// One sample's footprint for the index: anchor column, the two map rows and the 1-D weights
// (zero where the column / row lies outside the map), from the same arithmetic as
// decode_corners, so that wx*wy reproduces the corner weights of the other kernels bit for bit.
struct Footprint {
    int a;            // x0 + 1
    int y[2];
    float wx[2], wy[2];
};
__device__ __forceinline__ void decode_footprint(float cx, float cy, int W, int H, float hw, float hh, Footprint& f) {
    const float x = unnormalize(cx, hw), y = unnormalize(cy, hh);
    const float xf = floorf(x), yf = floorf(y);
    float fx = x - xf, fy = y - yf;
    const bool xr = (xf >= -2.0f) && (xf <= (float)W + 1.0f);
    const bool yr = (yf >= -2.0f) && (yf <= (float)H + 1.0f);
    const int x0 = xr ? (int)xf : -2, y0 = yr ? (int)yf : -2;
    if (!xr) fx = 0.0f;
    if (!yr) fy = 0.0f;
    const int x1 = x0 + 1, y1 = y0 + 1;
    f.wx[0] = (x0 >= 0 && x0 < W) ? 1.0f - fx : 0.0f;
    f.wx[1] = (x1 >= 0 && x1 < W) ? fx : 0.0f;
    f.wy[0] = (y0 >= 0 && y0 < H) ? 1.0f - fy : 0.0f;
    f.wy[1] = (y1 >= 0 && y1 < H) ? fy : 0.0f;
    f.a = x1;
    f.y[0] = y0;
    f.y[1] = y1;
}

// Shared memory: cnt[nhist][A] ints, then lens[A], part[NWARPS*32], bucket[nslab*kLenBuckets]
// ints.  (A template so that the header can be included by several translation units.)
template <int NWARPS>
__global__ void __launch_bounds__(NWARPS * 32) index_build_kernel(const IndexParams p) {
    static_assert(NWARPS >= 1 && NWARPS <= 32, "one warp scans the NWARPS*32 partial sums, NWARPS per lane");
    extern __shared__ __align__(16) unsigned char smem[];
    int* cnt = reinterpret_cast<int*>(smem);
    int* lens = cnt + p.nhist * p.A;       // first entry of every anchor's list, later its length
    int* part = lens + p.A;
    int* bucket = part + NWARPS * 32;

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
    // each of the first nhist warps owns a contiguous run of samples (a multiple of 32 of them)
    const int per_warp = ((nsamp + p.nhist * 32 - 1) / (p.nhist * 32)) * 32;
    const int wbeg = warp < p.nhist ? min(warp * per_warp, nsamp) : nsamp;
    const int wend = min(wbeg + per_warp, nsamp);
    int* mycnt = cnt + (warp < p.nhist ? warp : 0) * p.A;
    const int AW = p.W + 1;

    for (int i = threadIdx.x; i < p.nhist * p.A; i += blockDim.x) cnt[i] = 0;
    __syncthreads();

    // sample index (within the tile) -> coordinates; samples are ordered (query, s)
    auto coord_of = [&](int smp) -> float2 {
        const int ql = smp / p.S, s = smp - ql * p.S;
        const size_t row = ((((size_t)b * p.V + vq) * p.L + (l0 + ql)) * p.V + vk) * (size_t)p.S + s;
        return __ldg(reinterpret_cast<const float2*>(p.coords) + row);
    };
    // the entry of map row r (0, 1) of a footprint: present iff one of its two weights is not zero
    auto entry_of = [&](const Footprint& f, int r, float& wl, float& wr) -> int {
        wl = f.wx[0] * f.wy[r];
        wr = f.wx[1] * f.wy[r];
        if (wl == 0.0f && wr == 0.0f) return -1;
        return f.y[r] * AW + f.a;
    };

    // Both passes over the samples fetch the coordinates of kAhead steps (32 samples each) before
    // they work on the first: the loop is bound by the latency of those loads, not by their volume.
    constexpr int kAhead = 4;

    // pass 1: per-warp histogram of anchors
    for (int base = wbeg; base < wend; base += 32 * kAhead) {
        float2 c[kAhead];
#pragma unroll
        for (int u = 0; u < kAhead; ++u) {
            const int smp = base + u * 32 + lane;
            c[u] = smp < wend ? coord_of(smp) : make_float2(0.0f, 0.0f);
        }
#pragma unroll
        for (int u = 0; u < kAhead; ++u) {
            if (base + u * 32 + lane < wend) {
                Footprint f;
                decode_footprint(c[u].x, c[u].y, p.W, p.H, p.hw, p.hh, f);
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    float wl, wr;
                    const int a = entry_of(f, r, wl, wr);
                    if (a >= 0 && in_range(a, p.A, p.err)) atomicAdd(&mycnt[a], 1);
                }
            }
        }
    }
    __syncthreads();

    // pass 2: exclusive scan over anchors of the per-anchor totals -> row pointers, and
    // per-warp start offsets inside each anchor's list (warp order = canonical order)
    const int nthr = blockDim.x;
    const int chunk = (p.A + nthr - 1) / nthr;
    const int pbeg = min((int)threadIdx.x * chunk, p.A), pend = min(pbeg + chunk, p.A);
    int local = 0;
    for (int a = pbeg; a < pend; ++a)
        for (int w = 0; w < p.nhist; ++w) local += cnt[w * p.A + a];
    part[threadIdx.x] = local;
    __syncthreads();
    if (warp == 0) {
        // scan of the NWARPS*32 partial sums by one warp, NWARPS per lane
        int v[NWARPS], sum = 0;
#pragma unroll
        for (int i = 0; i < NWARPS; ++i) { v[i] = part[lane * NWARPS + i]; sum += v[i]; }
        int incl = sum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += n;
        }
        int run = incl - sum;
#pragma unroll
        for (int i = 0; i < NWARPS; ++i) { part[lane * NWARPS + i] = run; run += v[i]; }
    }
    __syncthreads();
    int run = part[threadIdx.x];
    for (int a = pbeg; a < pend; ++a) {
        lens[a] = run;
        for (int w = 0; w < p.nhist; ++w) {
            const int c = cnt[w * p.A + a];
            cnt[w * p.A + a] = run;
            run += c;
        }
    }
    for (int i = threadIdx.x; i < p.nslab * kLenBuckets; i += blockDim.x) bucket[i] = 0;
    __syncthreads();

    // pass 3: scatter in canonical order (32 samples at a time, map row 0 before map row 1),
    // ranks of equal anchors inside the warp from match_any
    uint4* entries = p.entries + (size_t)seg * (size_t)p.seg_entries;
    for (int base4 = wbeg; base4 < wend; base4 += 32 * kAhead) {
        float2 c[kAhead];
#pragma unroll
        for (int u = 0; u < kAhead; ++u) {
            const int smp = base4 + u * 32 + lane;
            c[u] = smp < wend ? coord_of(smp) : make_float2(0.0f, 0.0f);
        }
#pragma unroll
        for (int u = 0; u < kAhead; ++u) {
            const int base = base4 + u * 32;
            if (base >= wend) break;            // the same for the whole warp
            const int smp = base + lane;
            Footprint f;
            f.a = 0; f.y[0] = f.y[1] = 0;
            f.wx[0] = f.wx[1] = f.wy[0] = f.wy[1] = 0.0f;
            uint32_t roff = 0, soff = 0;
            if (smp < wend) {
                decode_footprint(c[u].x, c[u].y, p.W, p.H, p.hw, p.hh, f);
                // what the gather pass needs of the sample: where its query's row starts in the
                // tile and where its pair of scalars lies among the tile's, both in bytes
                roff = (uint32_t)(smp / p.S) * (uint32_t)p.rowb;
                soff = (uint32_t)smp * 8u;
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                float wl, wr;
                const int a = entry_of(f, r, wl, wr);
                const bool valid = a >= 0 && in_range(a, p.A, p.err);
                const unsigned vmask = __ballot_sync(0xffffffffu, valid);
                if (valid) {
                    const unsigned same = __match_any_sync(vmask, a);
                    const int leader = __ffs(same) - 1;
                    const int rank = __popc(same & ((1u << lane) - 1u));
                    int start = 0;
                    if (lane == leader) {
                        start = mycnt[a];
                        mycnt[a] = start + __popc(same);
                    }
                    start = __shfl_sync(same, start, leader);
                    if (in_range(start + rank, p.seg_entries, p.err))
                        entries[start + rank] = make_uint4(roff, soff, __float_as_uint(wl), __float_as_uint(wr));
                }
                __syncwarp();
            }
        }
    }
    __syncthreads();

    // pass 4: the work list.  Counting sort of the anchors by (slab of map rows, list length
    // descending); empty lists end up behind each slab's non-empty ones and are not written.
    // (Anchors of equal length land in arbitrary order: which group of lanes works on an anchor
    // does not change any sum.)
    const int rows_per_slab = (p.H + p.nslab - 1) / p.nslab;
    auto bucket_of = [&](int a, int len) -> int {
        const int slab = (a / AW) / rows_per_slab;
        return slab * kLenBuckets + (kLenBuckets - 1 - min(len, kLenBuckets - 1));
    };
    for (int a = pbeg; a < pend; ++a) {
        // the last histogram's cursor has run to the end of the anchor's list
        const int len = cnt[(p.nhist - 1) * p.A + a] - lens[a];
        atomicAdd(&bucket[bucket_of(a, len)], 1);
    }
    __syncthreads();
    {
        const int nb = p.nslab * kLenBuckets, per = (nb + nthr - 1) / nthr;   // buckets per thread
        const int b0 = min((int)threadIdx.x * per, nb), b1 = min(b0 + per, nb);
        int sum = 0;
        for (int i = b0; i < b1; ++i) sum += bucket[i];
        part[threadIdx.x] = sum;
        __syncthreads();
        if (warp == 0) {
            int v[NWARPS], tot = 0;
#pragma unroll
            for (int i = 0; i < NWARPS; ++i) { v[i] = part[lane * NWARPS + i]; tot += v[i]; }
            int incl = tot;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int n = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += n;
            }
            int r2 = incl - tot;
#pragma unroll
            for (int i = 0; i < NWARPS; ++i) { part[lane * NWARPS + i] = r2; r2 += v[i]; }
        }
        __syncthreads();
        int at = part[threadIdx.x];
        for (int i = b0; i < b1; ++i) {
            const int c = bucket[i];
            bucket[i] = at;
            at += c;
        }
        __syncthreads();
        if ((int)threadIdx.x < p.nslab) {
            const int first = bucket[threadIdx.x * kLenBuckets];
            p.sched_hdr[(size_t)seg * p.nslab + threadIdx.x] =
                make_int2(first, bucket[threadIdx.x * kLenBuckets + kLenBuckets - 1] - first);
        }
        __syncthreads();   // the headers are read before the cursors move
    }
    int4* sched = p.sched + (size_t)seg * p.A;
    for (int a = pbeg; a < pend; ++a) {
        const int beg = lens[a], end = cnt[(p.nhist - 1) * p.A + a];
        if (end == beg) continue;
        const int pos = atomicAdd(&bucket[bucket_of(a, end - beg)], 1);
        const int ay = a / AW, ax = a - ay * AW;
        if (in_range(pos, p.A, p.err)) sched[pos] = make_int4(ay * p.W + ax, beg, end, ax);
    }
}

struct GatherParams {
    const void* q;
    const void* dout;
    const float2* scal;
    const int4* sched;
    const int2* sched_hdr;
    const uint4* entries;
    // fp32 accumulators [B,V,Hh,L,D]: contributions a pixel receives as the left / right one of
    // an anchor.  (fp32 storage: the left maps are the dk/dv outputs themselves.)
    float* dk_left;
    float* dv_left;
    float* dk_right;
    float* dv_right;
    // where the finished maps go: dk/dv in the storage type and the optional mirrors (may be
    // another GPU's memory)
    void* dk;
    void* dv;
    void* dk_mirror;
    void* dv_mirror;
    int B, V, Hh, W, H, L, S;
    int tpv, QB;
    int seg_entries;
    int A;                // anchors per map: H*(W+1)
    int nslab;            // CTAs per (batch, head, key view); each takes a run of map rows
    int* err;
};

// Unpacking of one 32-bit word of two 16-bit elements: the low / high element as fp32.
// (bf16: byte permutes, which run on the integer pipe and leave the fma pipe to the fmas)
__device__ __forceinline__ float word_lo(uint32_t w, __nv_bfloat16*) { return __uint_as_float(__byte_perm(w, 0u, 0x1044)); }
__device__ __forceinline__ float word_hi(uint32_t w, __nv_bfloat16*) { return __uint_as_float(__byte_perm(w, 0u, 0x3244)); }
__device__ __forceinline__ float word_lo(uint32_t w, __half*) { return __half2float(__ushort_as_half((unsigned short)(w & 0xffffu))); }
__device__ __forceinline__ float word_hi(uint32_t w, __half*) { return __half2float(__ushort_as_half((unsigned short)(w >> 16))); }

// The accumulators of one anchor held by one lane: its EPL elements of the dK and dV rows of the
// left and of the right pixel.
//   16-bit storage: pairs (dK_e, dV_e), so that one packed fma serves both maps with the
//     multiplier pair (a*w, p*w) and the operand pair (q_e, dout_e), which the unpacking writes
//     side by side;
//   fp32 storage: pairs of neighbouring elements (as they lie in the loaded row) per map.
template <typename T, int D>
struct AnchorAcc {
    using RC = RowCfg<T, D>;
    static constexpr bool NARROW = sizeof(T) == 2;
    static constexpr int N = RC::EPL;   // float2 per side (both layouts)
    float2 left[N], right[N];

    __device__ __forceinline__ void clear() {
#pragma unroll
        for (int i = 0; i < N; ++i) left[i] = right[i] = make_float2(0.0f, 0.0f);
    }

    // One entry: rows of the entry's query at shared addresses q_row / do_row (this lane's first
    // vector), multipliers (aL, pL) for the left pixel and (aR, pR) for the right one.
    __device__ __forceinline__ void add(uint32_t q_row, uint32_t do_row, float aL, float pL, float aR, float pR) {
        constexpr int G = RC::G, CH = RC::CH;
        if constexpr (NARROW) {
            const float2 mL = make_float2(aL, pL), mR = make_float2(aR, pR);
#pragma unroll
            for (int ch = 0; ch < CH; ++ch) {
                const uint4 rq = lds128(q_row + (uint32_t)(ch * G) * 16u), rd = lds128(do_row + (uint32_t)(ch * G) * 16u);
                const uint32_t wq[4] = { rq.x, rq.y, rq.z, rq.w }, wd[4] = { rd.x, rd.y, rd.z, rd.w };
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 lo = make_float2(word_lo(wq[i], (T*)nullptr), word_lo(wd[i], (T*)nullptr));
                    const float2 hi = make_float2(word_hi(wq[i], (T*)nullptr), word_hi(wd[i], (T*)nullptr));
                    const int e = ch * 8 + 2 * i;
                    left[e] = __ffma2_rn(mL, lo, left[e]);
                    left[e + 1] = __ffma2_rn(mL, hi, left[e + 1]);
                    right[e] = __ffma2_rn(mR, lo, right[e]);
                    right[e + 1] = __ffma2_rn(mR, hi, right[e + 1]);
                }
            }
        } else {
            // layout per side: [ch][dK pair 0, dK pair 1, dV pair 0, dV pair 1]
            const float2 aL2 = make_float2(aL, aL), pL2 = make_float2(pL, pL);
            const float2 aR2 = make_float2(aR, aR), pR2 = make_float2(pR, pR);
#pragma unroll
            for (int ch = 0; ch < CH; ++ch) {
                float2 fq[2], fd[2];
                unpack16_pairs(lds128(q_row + (uint32_t)(ch * G) * 16u), fq, (T*)nullptr);
                unpack16_pairs(lds128(do_row + (uint32_t)(ch * G) * 16u), fd, (T*)nullptr);
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                    left[ch * 4 + k] = __ffma2_rn(aL2, fq[k], left[ch * 4 + k]);
                    left[ch * 4 + 2 + k] = __ffma2_rn(pL2, fd[k], left[ch * 4 + 2 + k]);
                    right[ch * 4 + k] = __ffma2_rn(aR2, fq[k], right[ch * 4 + k]);
                    right[ch * 4 + 2 + k] = __ffma2_rn(pR2, fd[k], right[ch * 4 + 2 + k]);
                }
            }
        }
    }

    // Adds one side to the rows of pixel `pix` of the dK / dV maps (this lane's elements).  Each
    // element of these maps has a single writer, so the reduction is only a store that needs no
    // read first.
    __device__ __forceinline__ void flush_side(const float2 (&acc)[N], float* dkmap, float* dvmap, int pix, int li) const {
        constexpr int G = RC::G, CH = RC::CH, EPV = RC::EPV;
#pragma unroll
        for (int ch = 0; ch < CH; ++ch) {
            const size_t off = (size_t)pix * D + (size_t)(ch * G + li) * EPV;
            if constexpr (NARROW) {
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                    const int e = ch * 8 + 4 * k;
                    red_global_add_v4(dkmap + off + 4 * k, acc[e].x, acc[e + 1].x, acc[e + 2].x, acc[e + 3].x);
                    red_global_add_v4(dvmap + off + 4 * k, acc[e].y, acc[e + 1].y, acc[e + 2].y, acc[e + 3].y);
                }
            } else {
                red_global_add_v4(dkmap + off, acc[ch * 4].x, acc[ch * 4].y, acc[ch * 4 + 1].x, acc[ch * 4 + 1].y);
                red_global_add_v4(dvmap + off, acc[ch * 4 + 2].x, acc[ch * 4 + 2].y, acc[ch * 4 + 3].x, acc[ch * 4 + 3].y);
            }
        }
    }
};

// After the last tile: the CTA adds the left and right maps of its map rows and hands the
// finished rows over: rounded to the storage type into dK/dV, and into the mirrors.  These
// stores are spread over the time the CTAs of the grid finish at.
template <typename T, int D>
__device__ __forceinline__ void gather_hand_over(const GatherParams& p, size_t map_row0, int pix_lo, int pix_hi) {
    using RC = RowCfg<T, D>;
    constexpr int EPV = RC::EPV, VEC = RC::VEC, ROWB = RC::ROWB;
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {
        const float* accl = (which ? p.dv_left : p.dk_left) + map_row0 * D;
        const float* accr = (which ? p.dv_right : p.dk_right) + map_row0 * D;
        char* o_loc = (char*)(which ? p.dv : p.dk) + map_row0 * ROWB;
        void* mir = which ? p.dv_mirror : p.dk_mirror;
        char* o_mir = mir ? (char*)mir + map_row0 * ROWB : nullptr;
        // one 16-byte vector of the storage type per thread and step
        const int nvec = (pix_hi - pix_lo) * VEC;
        for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
            const size_t e0 = (size_t)pix_lo * D + (size_t)i * EPV;
            float f[EPV];
#pragma unroll
            for (int k = 0; k < EPV / 4; ++k) {
                const float4 a = __ldcg(reinterpret_cast<const float4*>(accl + e0) + k);
                const float4 c = __ldcg(reinterpret_cast<const float4*>(accr + e0) + k);
                f[4 * k] = a.x + c.x; f[4 * k + 1] = a.y + c.y; f[4 * k + 2] = a.z + c.z; f[4 * k + 3] = a.w + c.w;
            }
            const uint4 packed = pack16(f, (T*)nullptr);
            const size_t o = (size_t)pix_lo * ROWB + (size_t)i * 16;
            stg128(o_loc + o, packed);
            if (o_mir) stg128(o_mir + o, packed);
        }
    }
}

// Entries travel from global memory to the lanes in chunks: the first kGatherChunk lanes of a
// group load one entry each (one coalesced request, issued a whole chunk ahead of its use) and
// park them in a small ring in shared memory, from which every lane of the group then reads
// them one by one.  Two chunk buffers per group, and 16 bytes of padding so that the groups of
// a warp, which tend to sit at the same position of their chunks, hit different banks.
template <int G>
struct GatherRing {
    static constexpr int CHUNK = G < 8 ? G : 8;
    static constexpr uint32_t STRIDE = 2u * CHUNK * 16u + 16u;   // bytes per group
};

// Shared memory of one tile: q rows and dout rows in the storage type ([QB, D] each), then
// the tile's scalars ([QB, S] float2), all three filled by bulk copies; then the mbarrier and
// the groups' entry rings.
template <typename T, int D>
__global__ void __launch_bounds__(sizeof(T) == 2 ? kGatherThreadsNarrow : kGatherThreadsFp32, 1)
bwd_gather_kernel(const GatherParams p) {
    using RC = RowCfg<T, D>;
    constexpr int G = RC::G, NG = RC::NG, ROWB = RC::ROWB;
    constexpr int CHUNK = GatherRing<G>::CHUNK;
    extern __shared__ __align__(128) unsigned char smem[];

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int g = lane / G, li = lane % G;
    const unsigned gmask = G == 32 ? 0xffffffffu : (((1u << (G & 31)) - 1u) << (g * G));
    // (nslab > 1: several CTAs share one (batch, head, key view) and split its map rows, which
    // evens out the last wave of a small grid; each still loads every tile)
    const int slab = blockIdx.x % p.nslab, unit = blockIdx.x / p.nslab;
    const int rows_per_slab = (p.H + p.nslab - 1) / p.nslab;
    const int y_lo = min(slab * rows_per_slab, p.H), y_hi = min(y_lo + rows_per_slab, p.H);
    const int ngroups = nw * NG, gid = warp * NG + g;
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
    const uint32_t ring = bar + 16u + (uint32_t)gid * GatherRing<G>::STRIDE;

    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
        fence_proxy_async();
    }
    __syncthreads();

    const size_t map_row0 = (((size_t)b * p.V + vk) * p.Hh + h) * (size_t)p.L;
    float* dkl = p.dk_left + map_row0 * D;
    float* dvl = p.dv_left + map_row0 * D;
    float* dkr = p.dk_right + map_row0 * D;
    float* dvr = p.dv_right + map_row0 * D;
    unsigned chunk_no = 0;   // alternates the ring's two buffers; runs on across anchors and tiles

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
            const int2 hdr = __ldg(p.sched_hdr + seg * p.nslab + slab);
            const int4* sched = p.sched + seg * (size_t)p.A + hdr.x;
            const int nwork = hdr.y;
            const uint4* entries = p.entries + seg * (size_t)p.seg_entries;
            // The work list is sorted by list length: the groups of a warp, which take neighbouring
            // records, run loops of (nearly) equal length, and dealing the list out back and forth
            // (0..n-1, n-1..0, ...) gives every group the same total.  The walk is software-
            // pipelined: the record after next and the first chunk of the next record's entries
            // are requested before the current record's entries are processed, so that their L2
            // latency hides behind that work.
            const int back = ngroups - 1 - gid;
            int4 rec = make_int4(0, 0, 0, 0), nrec = rec;
            if (gid < nwork) rec = __ldg(sched + gid);
            if (ngroups + back < nwork) nrec = __ldg(sched + ngroups + back);
            uint4 first = make_uint4(0, 0, 0, 0);
            if (li < CHUNK && rec.y + li < rec.z) first = __ldg(entries + rec.y + li);
            for (int round = 0; round * ngroups < nwork; ++round) {
                int4 n2rec = make_int4(0, 0, 0, 0);
                {
                    const int pos2 = (round + 2) * ngroups + (round & 1 ? back : gid);
                    if (pos2 < nwork) n2rec = __ldg(sched + pos2);
                }
                uint4 nfirst = make_uint4(0, 0, 0, 0);
                if (li < CHUNK && nrec.y + li < nrec.z) nfirst = __ldg(entries + nrec.y + li);
                const int beg = rec.y, end = rec.z;
                if (end > beg) {
                    AnchorAcc<T, D> acc;
                    acc.clear();
                    uint4 mine = first;   // this lane's entry of the chunk about to be processed
                    for (int e0 = beg; e0 < end; e0 += CHUNK, ++chunk_no) {
                        const uint32_t buf = ring + (chunk_no & 1u) * (uint32_t)(CHUNK * 16);
                        if (li < CHUNK) sts128(buf + (uint32_t)li * 16u, mine);
                        __syncwarp(gmask);
                        if (li < CHUNK && e0 + CHUNK + li < end) mine = __ldg(entries + e0 + CHUNK + li);
                        auto one = [&](int i) {
                            const uint4 ent = lds128(buf + (uint32_t)i * 16u);
                            if (!in_range(ent.x, (long long)p.QB * ROWB, p.err) || !in_range(ent.y, (long long)p.QB * p.S * 8, p.err))
                                return;
                            float2 sc;
                            asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(sc.x), "=f"(sc.y) : "r"(sc_s + ent.y));
                            const float wl = __uint_as_float(ent.z), wr = __uint_as_float(ent.w);
                            acc.add(q_s + ent.x, do_s + ent.x, sc.x * wl, sc.y * wl, sc.x * wr, sc.y * wr);
                        };
                        const int n = end - e0;
                        if (n >= CHUNK) {
                            // a full chunk: straight-line code, no tests between the entries
#pragma unroll
                            for (int i = 0; i < CHUNK; ++i) one(i);
                        } else {
                            for (int i = 0; i < n; ++i) one(i);
                        }
                    }
                    const int pix = rec.x, ax = rec.w;  // the right pixel; the left one is pix - 1
                    if (ax > 0 && in_range(pix - 1, p.L, p.err)) acc.flush_side(acc.left, dkl, dvl, pix - 1, li);
                    if (ax < p.W && in_range(pix, p.L, p.err)) acc.flush_side(acc.right, dkr, dvr, pix, li);
                }
                rec = nrec;
                nrec = n2rec;
                first = nfirst;
            }
        }
        // every group is done with the tile before its buffers are refilled
        if (__syncthreads_or(ok ? 0 : 1)) return;
    }

    // the additions of all groups reach memory before any thread reads the maps back
    __threadfence();
    __syncthreads();
    gather_hand_over<T, D>(p, map_row0, y_lo * p.W, y_hi * p.W);
}

}  // namespace dsdpa

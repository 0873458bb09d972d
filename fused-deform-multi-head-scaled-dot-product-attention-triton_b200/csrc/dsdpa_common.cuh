// Shared device helpers for the deformable-SDPA kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "../../include/dsdpa.h"

namespace dsdpa {

constexpr int kSMs = 148;                    // B200
constexpr int kSmemMax = 232448;             // 227 KB opt-in shared memory per CTA
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr unsigned kWaitLimit = 1u << 22;    // polls of an mbarrier before a kernel gives up

// ---------------------------------------------------------------------------------
// How one row of D elements of type T is spread over the lanes of a warp:
// a row is VEC 16-byte vectors; G = min(VEC, 32) lanes ("a group") own one row at a
// time, lane i of the group holding vectors i, i+G, ...  A warp is NG = 32/G groups.
// ---------------------------------------------------------------------------------
template <typename T, int D>
struct RowCfg {
    static constexpr int EPV = 16 / (int)sizeof(T);  // elements per 16-byte vector
    static constexpr int VEC = D / EPV;
    static constexpr int G = VEC < 32 ? VEC : 32;
    static constexpr int CH = VEC / G;               // vectors per lane
    static constexpr int NG = 32 / G;
    static constexpr int EPL = EPV * CH;             // elements per lane
    static constexpr int ROWB = D * (int)sizeof(T);
    static_assert(D % EPV == 0 && VEC >= 2, "head dim too small for 16-byte vectors");
    static_assert(VEC % G == 0, "row does not split evenly over the group");
};

template <typename T> struct DtypeOf;
template <> struct DtypeOf<float> { static constexpr int value = DSDPA_F32; };
template <> struct DtypeOf<__nv_bfloat16> { static constexpr int value = DSDPA_BF16; };
template <> struct DtypeOf<__half> { static constexpr int value = DSDPA_F16; };

// ---- 16-byte vector <-> fp32 lanes -----------------------------------------------
__device__ __forceinline__ void unpack16(const uint4& r, float (&f)[4], float*) {
    f[0] = __uint_as_float(r.x); f[1] = __uint_as_float(r.y);
    f[2] = __uint_as_float(r.z); f[3] = __uint_as_float(r.w);
}
__device__ __forceinline__ void unpack16(const uint4& r, float (&f)[8], __nv_bfloat16*) {
    const uint32_t w[4] = { r.x, r.y, r.z, r.w };
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
__device__ __forceinline__ void unpack16(const uint4& r, float (&f)[8], __half*) {
    const uint32_t w[4] = { r.x, r.y, r.z, r.w };
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
        float2 t = __half22float2(h);
        f[2 * i] = t.x; f[2 * i + 1] = t.y;
    }
}

// The same, as fp32 PAIRS (operands of fma.rn.f32x2): element 2i in .x, 2i+1 in .y.
__device__ __forceinline__ void unpack16_pairs(const uint4& r, float2 (&f)[2], float*) {
    f[0] = make_float2(__uint_as_float(r.x), __uint_as_float(r.y));
    f[1] = make_float2(__uint_as_float(r.z), __uint_as_float(r.w));
}
__device__ __forceinline__ void unpack16_pairs(const uint4& r, float2 (&f)[4], __nv_bfloat16*) {
    const uint32_t w[4] = { r.x, r.y, r.z, r.w };
#pragma unroll
    for (int i = 0; i < 4; ++i)
        f[i] = make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
}
__device__ __forceinline__ void unpack16_pairs(const uint4& r, float2 (&f)[4], __half*) {
    const uint32_t w[4] = { r.x, r.y, r.z, r.w };
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
}

__device__ __forceinline__ uint4 pack16(const float (&f)[4], float*) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
}
__device__ __forceinline__ uint4 pack16(const float (&f)[8], __nv_bfloat16*) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);  // one rounding, fp32 -> bf16
        w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ uint4 pack16(const float (&f)[8], __half*) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
        w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// ---- loads -------------------------------------------------------------------------
__device__ __forceinline__ uint4 lds128(uint32_t saddr) {
    uint4 r;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(saddr));
    return r;
}
__device__ __forceinline__ uint4 ldg128_nc(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}
__device__ __forceinline__ uint4 ldg128_stream(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}
__device__ __forceinline__ void stg128(void* p, const uint4& r) {
    asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" :: "l"(p), "r"(r.x), "r"(r.y), "r"(r.z), "r"(r.w) : "memory");
}
__device__ __forceinline__ void sts128(uint32_t saddr, const uint4& r) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" :: "r"(saddr), "r"(r.x), "r"(r.y), "r"(r.z), "r"(r.w) : "memory");
}

// ---- reductions to memory ---------------------------------------------------------------
__device__ __forceinline__ void red_global_add_v4(float* p, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};" :: "l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void red_shared_add(uint32_t saddr, float a) {
    asm volatile("red.shared.add.f32 [%0], %1;" :: "r"(saddr), "f"(a) : "memory");
}

// ---- dot products of 16-bit vectors with fp32 accumulation (sm_100 mixed-precision fma) -----
// fma.rn.f32.{bf16,f16} multiplies two 16-bit operands exactly (8+8 resp. 11+11 mantissa bits fit
// in fp32) and adds an fp32 accumulator: one instruction per element, against two (unpack, fma) on
// the fp32 path, and no rounding of the operands.
__device__ __forceinline__ float fma_mixed(uint16_t a, uint16_t b, float c, __nv_bfloat16*) {
    float d;
    asm("fma.rn.f32.bf16 %0, %1, %2, %3;" : "=f"(d) : "h"(a), "h"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float fma_mixed(uint16_t a, uint16_t b, float c, __half*) {
    float d;
    asm("fma.rn.f32.f16 %0, %1, %2, %3;" : "=f"(d) : "h"(a), "h"(b), "f"(c));
    return d;
}
// acc + sum over the eight 16-bit elements of a and b
template <typename T>
__device__ __forceinline__ float dot16(const uint4& a, const uint4& b, float acc) {
    const uint32_t aw[4] = { a.x, a.y, a.z, a.w }, bw[4] = { b.x, b.y, b.z, b.w };
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint16_t alo, ahi, blo, bhi;
        asm("mov.b32 {%0, %1}, %2;" : "=h"(alo), "=h"(ahi) : "r"(aw[i]));
        asm("mov.b32 {%0, %1}, %2;" : "=h"(blo), "=h"(bhi) : "r"(bw[i]));
        acc = fma_mixed(alo, blo, acc, (T*)nullptr);
        acc = fma_mixed(ahi, bhi, acc, (T*)nullptr);
    }
    return acc;
}

// Two fp32 scalars rounded to the 16-bit storage type (round to nearest even), returned as the
// two 16-bit operands the mixed-precision fma takes.
__device__ __forceinline__ void round_pair16(float a, float b, uint16_t& ra, uint16_t& rb, __nv_bfloat16*) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));   // upper half <- b, lower <- a
    asm("mov.b32 {%0, %1}, %2;" : "=h"(ra), "=h"(rb) : "r"(r));
}
__device__ __forceinline__ void round_pair16(float a, float b, uint16_t& ra, uint16_t& rb, __half*) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
    asm("mov.b32 {%0, %1}, %2;" : "=h"(ra), "=h"(rb) : "r"(r));
}
// acc[0..3] += s * row for the eight 16-bit elements of `row` (pairs as unpack16_pairs orders them):
// s is a 16-bit scalar, products are exact, the sums fp32.
template <typename T>
__device__ __forceinline__ void axpy16(uint16_t s, const uint4& row, float2* acc) {
    const uint32_t w[4] = { row.x, row.y, row.z, row.w };
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint16_t lo, hi;
        asm("mov.b32 {%0, %1}, %2;" : "=h"(lo), "=h"(hi) : "r"(w[i]));
        acc[i].x = fma_mixed(s, lo, acc[i].x, (T*)nullptr);
        acc[i].y = fma_mixed(s, hi, acc[i].y, (T*)nullptr);
    }
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

// ---- mbarrier + 1-D bulk copy (TMA without a tensor map, no multicast) -----------
__device__ __forceinline__ void mbar_init(uint32_t bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, unsigned parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: returns false (after recording the fact) instead of spinning forever.
// `err` points at the library's per-device error word (read back by dsdpa_device_error()).
// The error word holds the first thing a kernel had to report: kErrTimeout (a wait ran out) or,
// in builds with -DDSDPA_BOUNDS_CHECK, kErrBounds (an index out of range; the access was skipped).
constexpr int kErrTimeout = 1;
constexpr int kErrBounds = 2;
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, unsigned parity, int* err, unsigned limit = kWaitLimit) {
    for (unsigned i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    atomicCAS(err, 0, kErrTimeout);
    return false;
}

// Checked debug build (-DDSDPA_BOUNDS_CHECK): every index the kernels compute for a gathered
// pixel row, an index entry or a shared-memory record is tested against its range before use;
// a violation is recorded in the error word and the access is skipped (the value reads as
// zero, a store is dropped), nothing traps.  In the normal build the test folds away.
#ifdef DSDPA_BOUNDS_CHECK
constexpr bool kBoundsCheck = true;
#else
constexpr bool kBoundsCheck = false;
#endif
__device__ __forceinline__ bool in_range(long long idx, long long n, int* err) {
    if (!kBoundsCheck) return true;
    if (idx >= 0 && idx < n) return true;
    atomicCAS(err, 0, kErrBounds);
    return false;
}
// dst: shared address, src: global address, both 16-byte aligned; bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, unsigned bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// One thread copies `bytes` (multiple of 16) in pieces, all completing on `bar`.
__device__ __forceinline__ void bulk_g2s_chunked(uint32_t dst, const char* src, unsigned bytes, uint32_t bar) {
    constexpr unsigned kPiece = 32768;
    for (unsigned off = 0; off < bytes; off += kPiece) {
        unsigned n = bytes - off < kPiece ? bytes - off : kPiece;
        bulk_g2s(dst + off, src + off, n, bar);
    }
}

// The K and V maps of one key view into a stage buffer ([K map][V map]) by one thread.  They
// complete on separate barriers, K on `bar` and V on `bar + 8` (an mbarrier counts up to 2^20-1
// bytes per phase, one map each keeps larger maps stageable).
__device__ __forceinline__ void stage_maps(uint32_t dst, const char* ksrc, const char* vsrc, unsigned map_bytes,
                                           uint32_t bar) {
    fence_proxy_async();
    mbar_expect_tx(bar, map_bytes);
    bulk_g2s_chunked(dst, ksrc, map_bytes, bar);
    mbar_expect_tx(bar + 8u, map_bytes);
    bulk_g2s_chunked(dst + map_bytes, vsrc, map_bytes, bar + 8u);
}

// ---- sampling-coordinate decode --------------------------------------------------
// One sample of one query: the four corner pixels of the bilinear footprint and their
// weights.  A corner outside the map keeps a clamped (valid) pixel index and gets
// weight 0, which is the reference's zero padding per corner (ops/torch.py:14-15,
// grid_sample defaults); the Triton kernel's whole-sample mask and edge clamp
// (ops/triton.py:129, 135-136) are deliberately not reproduced.
struct Corners {
    int pix[4];    // y0*W+x0, y0*W+x1, y1*W+x0, y1*W+x1 (clamped into the map)
    float w[4];    // weights, zero for corners outside the map
};

// Pixel position as ATen's CPU grid sampler computes it for align_corners=True from
// grid = c*2-1 (ops/torch.py:14): x = (grid + 1) * ((W-1)/2), each step rounded.
__device__ __forceinline__ float unnormalize(float c, float half_extent) {
    float g = __fadd_rn(__fmul_rn(c, 2.0f), -1.0f);
    return __fmul_rn(__fadd_rn(g, 1.0f), half_extent);
}

__device__ __forceinline__ void decode_corners(float cx, float cy, int W, int H, float hw, float hh,
                                               Corners& c, float& fx, float& fy) {
    float x = unnormalize(cx, hw), y = unnormalize(cy, hh);
    float xf = floorf(x), yf = floorf(y);
    fx = x - xf;
    fy = y - yf;
    // keep the int conversion in range for huge or non-finite coordinates
    bool xr = (xf >= -2.0f) && (xf <= (float)W + 1.0f);
    bool yr = (yf >= -2.0f) && (yf <= (float)H + 1.0f);
    int x0 = xr ? (int)xf : -2, y0 = yr ? (int)yf : -2;
    if (!xr) fx = 0.0f;
    if (!yr) fy = 0.0f;
    int x1 = x0 + 1, y1 = y0 + 1;
    float wx0 = (x0 >= 0 && x0 < W) ? 1.0f - fx : 0.0f;
    float wx1 = (x1 >= 0 && x1 < W) ? fx : 0.0f;
    float wy0 = (y0 >= 0 && y0 < H) ? 1.0f - fy : 0.0f;
    float wy1 = (y1 >= 0 && y1 < H) ? fy : 0.0f;
    int x0c = min(max(x0, 0), W - 1), x1c = min(max(x1, 0), W - 1);
    int y0c = min(max(y0, 0), H - 1), y1c = min(max(y1, 0), H - 1);
    c.pix[0] = y0c * W + x0c; c.pix[1] = y0c * W + x1c;
    c.pix[2] = y1c * W + x0c; c.pix[3] = y1c * W + x1c;
    c.w[0] = wx0 * wy0; c.w[1] = wx1 * wy0; c.w[2] = wx0 * wy1; c.w[3] = wx1 * wy1;
}

// Sum over the G lanes of a group (G a power of two <= 32); every lane gets the sum.
template <int G>
__device__ __forceinline__ float group_sum(float x) {
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

}  // namespace dsdpa

// Bandwidth probes of the benchmark (libdsdpa_probes.so): roofline denominators measured on
// the device at hand.  Not part of the product library: nothing in libdeform_sdpa.so calls or
// links this file.
//
// Every probe runs a read-only kernel on the given stream `iters` times after one warm-up,
// times it with CUDA events on that stream, synchronises and returns GB/s.  Status: 0 = ok,
// 1 = bad argument, 2 = CUDA error (the cudaError_t is returned through *cuda_error).
#include <cuda_runtime.h>
#include <stdint.h>

#include "../dsdpa_common.cuh"

namespace {

using dsdpa::lds128;
using dsdpa::ldg128_nc;
using dsdpa::ldg128_stream;
using dsdpa::sts128;
using dsdpa::smem_addr;

constexpr int kSMs = 148;
constexpr uint32_t kWindow = 65536;        // bytes of shared memory the patterns roam over
constexpr uint32_t kSlack = 8192;          // room behind the window for spans that start near its end
__device__ unsigned g_sink;                // never read; keeps the loads alive

// ---- L2: every CTA sweeps the whole (L2-resident) buffer from its own offset ---------------
__global__ void __launch_bounds__(1024, 1) l2_kernel(const uint4* __restrict__ buf, size_t nvec) {
    const size_t start = (size_t)blockIdx.x * 4099u * 1024u % nvec;
    unsigned acc = 0;
    const size_t stride = blockDim.x;
    for (size_t i = threadIdx.x; i + 3 * stride < nvec; i += 4 * stride) {
        size_t a = start + i; if (a >= nvec) a -= nvec;
        size_t b = start + i + stride; if (b >= nvec) b -= nvec;
        size_t c = start + i + 2 * stride; if (c >= nvec) c -= nvec;
        size_t d = start + i + 3 * stride; if (d >= nvec) d -= nvec;
        const uint4 x0 = ldg128_stream(buf + a), x1 = ldg128_stream(buf + b);
        const uint4 x2 = ldg128_stream(buf + c), x3 = ldg128_stream(buf + d);
        acc ^= x0.x ^ x0.w ^ x1.y ^ x1.z ^ x2.x ^ x2.w ^ x3.y ^ x3.z;
    }
    if (acc == 0x9e3779b9u) g_sink = acc;
}

// ---- shared memory: 128-bit loads, one access pattern per instantiation ---------------------
// A "unit" is a run of UNIT consecutive lanes that read UNIT*16 contiguous bytes; the units of
// a warp read unrelated places.  ALIGN is what the start of a unit's span is aligned to; with
// ODD the start is an odd multiple of ALIGN (aligned to ALIGN but never to 2*ALIGN).
//   UNIT=32 ALIGN=512        a warp reads one 512-byte line (conflict-free streaming)
//   UNIT=8  ALIGN=128        four unrelated 128-byte rows per instruction (a row gather)
//   UNIT=16 ALIGN=256        two unrelated 256-byte-aligned spans (a K|V merged row, or an
//                            x0/x0+1 corner pair with even x0)
//   UNIT=16 ALIGN=128 ODD    two unrelated 256-byte spans that straddle a 256-byte boundary
//                            (a corner pair with odd x0)
//   UNIT=32 ALIGN=128 ODD    one 512-byte span at 128-byte alignment (a corner pair of
//                            merged K|V rows)
//   CORNERS                  the four groups of eight lanes read rows r, r+1, r+W, r+W+1 of a
//                            28-pixel-wide map: the four corners of one bilinear sample
template <int UNIT, int ALIGN, bool ODD, bool CORNERS>
__global__ void __launch_bounds__(1024, 1) smem_pattern_kernel(int rounds) {
    extern __shared__ __align__(1024) unsigned char smem[];
    const uint32_t base = smem_addr(smem);
    for (uint32_t o = threadIdx.x * 16u; o < kWindow + kSlack; o += blockDim.x * 16u)
        sts128(base + o, make_uint4(o, o + 1, o + 2, o + 3));
    __syncthreads();
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t unit = threadIdx.x / UNIT;                 // the same for all lanes of a unit
    uint32_t within = (lane % UNIT) * 16u;
    if (CORNERS) within = (lane & 7u) * 16u + ((lane >> 3) & 1u) * 128u + (lane >> 4) * 28u * 128u;
    // eight start offsets per unit, fixed for the run; every round moves them all by the same
    // multiple of 2*ALIGN, which keeps alignment class and parity
    uint32_t off[8];
    uint32_t state = unit * 2654435761u + 12345u;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        state = state * 1664525u + 1013904223u;
        uint32_t o = ((state >> 10) % (kWindow / (2u * ALIGN))) * (2u * ALIGN);
        if (ODD) o += ALIGN;
        off[u] = o;
    }
    const uint32_t step = 2u * ALIGN * 37u;
    unsigned acc = 0;
    uint32_t shift = 0;
    for (int r = 0; r < rounds; ++r) {
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const uint4 x = lds128(base + ((off[u] + shift) & (kWindow - 1u)) + within);
            acc ^= x.x ^ x.y ^ x.z ^ x.w;
        }
        shift += step;
    }
    if (acc == 0x9e3779b9u) g_sink = acc;
}

// ---- L1: every group of eight lanes reads a 128-byte row of a small global buffer through
// the read-only path; the buffer (64 KB) stays in every SM's L1, so this is the ceiling of a
// row gather whose rows hit L1 ---------------------------------------------------------------
__global__ void __launch_bounds__(256, 4) l1_rows_kernel(const unsigned char* __restrict__ buf, int rounds) {
    const uint32_t unit = threadIdx.x / 8u + blockIdx.x * 32u;
    const uint32_t within = (threadIdx.x & 7u) * 16u;
    uint32_t off[8];
    uint32_t state = unit * 2654435761u + 12345u;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        state = state * 1664525u + 1013904223u;
        off[u] = ((state >> 10) % (kWindow / 128u)) * 128u;
    }
    unsigned acc = 0;
    uint32_t shift = 0;
    for (int r = 0; r < rounds; ++r) {
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const uint4 x = ldg128_nc(buf + ((off[u] + shift) & (kWindow - 1u)) + within);
            acc ^= x.x ^ x.y ^ x.z ^ x.w;
        }
        shift += 128u * 37u;
    }
    if (acc == 0x9e3779b9u) g_sink = acc;
}

struct Timer {
    cudaEvent_t a = nullptr, b = nullptr;
    cudaError_t begin() {
        cudaError_t e = cudaEventCreate(&a);
        if (e != cudaSuccess) return e;
        return cudaEventCreate(&b);
    }
    ~Timer() {
        if (a) cudaEventDestroy(a);
        if (b) cudaEventDestroy(b);
    }
};

template <typename Launch>
int time_it(cudaStream_t s, int iters, double bytes_per_iter, double* gbps, int* cuda_error, Launch launch) {
    Timer t;
    cudaError_t e = t.begin();
    if (e == cudaSuccess) {
        launch();  // warm-up
        cudaEventRecord(t.a, s);
        for (int i = 0; i < iters; ++i) launch();
        cudaEventRecord(t.b, s);
        e = cudaEventSynchronize(t.b);
    }
    float ms = 0.0f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, t.a, t.b);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) {
        if (cuda_error) *cuda_error = (int)e;
        (void)cudaGetLastError();
        return 2;
    }
    *gbps = bytes_per_iter * iters / ((double)ms * 1e-3) / 1e9;
    return 0;
}

template <int UNIT, int ALIGN, bool ODD, bool CORNERS>
int run_pattern(cudaStream_t s, int iters, double* gbps, int* cuda_error) {
    auto kern = smem_pattern_kernel<UNIT, ALIGN, ODD, CORNERS>;
    const int smem = (int)(kWindow + kSlack);
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) {
        if (cuda_error) *cuda_error = (int)e;
        return 2;
    }
    const int rounds = 4096;
    return time_it(s, iters, (double)rounds * 8.0 * 16.0 * 1024.0 * kSMs, gbps, cuda_error,
                   [&] { kern<<<kSMs, 1024, smem, s>>>(rounds); });
}

}  // namespace

extern "C" {

// Every SM reads a `bytes`-sized buffer (<= L2 size, caller-provided, 16-byte aligned) with
// 128-bit read-only loads that do not allocate in L1.
int dsdpa_probe_l2_read_bandwidth(const void* buffer, size_t bytes, int iters, int device, void* stream, double* gbps,
                                  int* cuda_error) {
    if (!buffer || !gbps || ((uintptr_t)buffer & 15u) || bytes < (1u << 20) || iters <= 0) return 1;
    if (cudaSetDevice(device) != cudaSuccess) return 1;
    const size_t nvec = bytes / 16 / 4096 * 4096;
    cudaStream_t s = (cudaStream_t)stream;
    return time_it(s, iters, (double)nvec * 16.0 * kSMs, gbps, cuda_error,
                   [&] { l2_kernel<<<kSMs, 1024, 0, s>>>((const uint4*)buffer, nvec); });
}

// Shared-memory read bandwidth of one access pattern (see smem_pattern_kernel):
//   0 contiguous 512-byte warp lines      1 four unrelated 128-byte rows
//   2 two 256-byte-aligned spans          3 two 256-byte spans across a 256-byte boundary
//   4 one 512-byte span at 128-byte alignment
//   5 the four corner rows of one sample (r, r+1, r+W, r+W+1)
int dsdpa_probe_shared_pattern(int pattern, int iters, int device, void* stream, double* gbps, int* cuda_error) {
    if (!gbps || iters <= 0) return 1;
    if (cudaSetDevice(device) != cudaSuccess) return 1;
    cudaStream_t s = (cudaStream_t)stream;
    switch (pattern) {
        case 0: return run_pattern<32, 512, false, false>(s, iters, gbps, cuda_error);
        case 1: return run_pattern<8, 128, false, false>(s, iters, gbps, cuda_error);
        case 2: return run_pattern<16, 256, false, false>(s, iters, gbps, cuda_error);
        case 3: return run_pattern<16, 128, true, false>(s, iters, gbps, cuda_error);
        case 4: return run_pattern<32, 128, true, false>(s, iters, gbps, cuda_error);
        case 5: return run_pattern<32, 128, false, true>(s, iters, gbps, cuda_error);
        default: return 1;
    }
}

// Row gather served by L1: `buffer` is a 64 KB global buffer (16-byte aligned).
int dsdpa_probe_l1_row_gather_bandwidth(const void* buffer, int iters, int device, void* stream, double* gbps,
                                        int* cuda_error) {
    if (!buffer || !gbps || ((uintptr_t)buffer & 15u) || iters <= 0) return 1;
    if (cudaSetDevice(device) != cudaSuccess) return 1;
    cudaStream_t s = (cudaStream_t)stream;
    const int rounds = 2048, ctas = kSMs * 4;
    return time_it(s, iters, (double)rounds * 8.0 * 16.0 * 256.0 * ctas, gbps, cuda_error,
                   [&] { l1_rows_kernel<<<ctas, 256, 0, s>>>((const unsigned char*)buffer, rounds); });
}

}  // extern "C"

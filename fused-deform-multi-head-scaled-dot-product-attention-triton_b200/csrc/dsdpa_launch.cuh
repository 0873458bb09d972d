// Launch dispatch: (dtype, head dim, slots, variant) -> kernel instantiation.
// The instantiations live in one translation unit per storage type and direction
// (dsdpa_inst_*.cu) so that they compile in parallel; this header is what they share
// with the C-ABI translation unit.
#pragma once

#include "dsdpa_bwd.cuh"
#include "dsdpa_bwd2.cuh"
#include "dsdpa_plan.h"

namespace dsdpa {

template <typename T>
cudaError_t launch_forward(const FwdParams& p, const TilePlan& plan, int D, cudaStream_t stream);
// two_pass: the kernel writes per-sample scalars instead of scattering (pass A)
template <typename T>
cudaError_t launch_backward_main(const BwdParams& p, const TilePlan& plan, int D, bool two_pass, bool dcoords,
                                 cudaStream_t stream);
template <typename T>
cudaError_t launch_backward_gather(const GatherParams& p, const GatherPlan& plan, int D, cudaStream_t stream);
template <typename T>
cudaError_t launch_cast_from_f32(const float* src, void* dst, size_t n, cudaStream_t stream);

// Thread limits the variants are compiled for (the plan must stay within them).
constexpr int kStagedMaxThreads = 512;
constexpr int kL2MaxThreads = 256;
// CTAs per SM the variants that gather from L1/L2 are compiled for (they hide latency with warps)
#ifndef DSDPA_L2_MIN_BLOCKS
#define DSDPA_L2_MIN_BLOCKS 2
#endif
constexpr int kL2MinBlocks = DSDPA_L2_MIN_BLOCKS;

namespace detail {

// Opt the kernel in to the full 227 KB of dynamic shared memory, once per device.
// `done` must be a flag array owned by the calling instantiation: the kernels of one
// family all share a function-pointer type, so a static in here would be shared too.
template <typename K>
inline cudaError_t allow_big_smem(K kern, bool (&done)[64]) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64 && done[dev]) return cudaSuccess;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax);
    if (e == cudaSuccess && dev >= 0 && dev < 64) done[dev] = true;
    return e;
}

template <typename T, int D, int NQ, bool STAGED, bool RW, bool TAILS, int MAXT = (STAGED ? kStagedMaxThreads : kL2MaxThreads)>
inline cudaError_t fwd_launch(const FwdParams& p, const TilePlan& plan, cudaStream_t stream) {
    auto kern = fwd_kernel<T, D, NQ, STAGED, MAXT, STAGED ? 1 : kL2MinBlocks, RW, TAILS>;
    if (plan.nw * 32 > MAXT) return cudaErrorInvalidValue;
    static bool done[64] = {};  // a benign race at worst repeats the attribute call
    cudaError_t e = allow_big_smem(kern, done);
    if (e != cudaSuccess) return e;
    kern<<<(unsigned)plan.ctas, plan.nw * 32, plan.smem, stream>>>(p);
    return cudaGetLastError();
}

// Samples come to a group in chunks of G (its lane count) and are taken UMAX at a time: when
// every chunk is whole batches the kernel without the tail code runs (it pads an incomplete
// batch instead, which then never happens).
template <typename T, int D, int NQ, bool STAGED, bool RW = false>
inline cudaError_t fwd_one(const FwdParams& p, const TilePlan& plan, cudaStream_t stream) {
    constexpr int G = RowCfg<T, D>::G;
    constexpr int UMAX = STAGED ? DSDPA_FWD_UNROLL : DSDPA_FWD_UNROLL_L2;
    const bool whole = G % UMAX == 0 && p.S % UMAX == 0;
    return whole ? fwd_launch<T, D, NQ, STAGED, RW, false>(p, plan, stream)
                 : fwd_launch<T, D, NQ, STAGED, RW, true>(p, plan, stream);
}

template <typename T, int D>
inline cudaError_t fwd_d(const FwdParams& p, const TilePlan& plan, cudaStream_t stream) {
    if constexpr (sizeof(T) == 2) {
        if (plan.rounded_weights) {
            if (!plan.staged) return fwd_one<T, D, 1, false, true>(p, plan, stream);
            switch (plan.nq) {
                case 1: return fwd_one<T, D, 1, true, true>(p, plan, stream);
                case 2: return fwd_one<T, D, 2, true, true>(p, plan, stream);
                default: return cudaErrorInvalidValue;
            }
        }
    }
    if (!plan.staged) return fwd_one<T, D, 1, false>(p, plan, stream);
    switch (plan.nq) {
        case 1: return fwd_one<T, D, 1, true>(p, plan, stream);
        case 2: return fwd_one<T, D, 2, true>(p, plan, stream);
        default: return cudaErrorInvalidValue;
    }
}

template <typename T, int D, int NQ, bool STAGED, bool PRIV, bool TWOPASS, bool DCOORDS = false>
inline cudaError_t bwd_one(const BwdParams& p, const TilePlan& plan, cudaStream_t stream) {
    auto kern = bwd_scatter_kernel<T, D, NQ, STAGED, PRIV, TWOPASS, DCOORDS,
                                   STAGED ? kStagedMaxThreads : kL2MaxThreads, STAGED ? 1 : kL2MinBlocks>;
    static bool done[64] = {};
    cudaError_t e = allow_big_smem(kern, done);
    if (e != cudaSuccess) return e;
    kern<<<(unsigned)plan.ctas, plan.nw * 32, plan.smem, stream>>>(p);
    return cudaGetLastError();
}

template <typename T, int D>
inline cudaError_t bwd_d(const BwdParams& p, const TilePlan& plan, bool two_pass, bool dcoords, cudaStream_t stream) {
    if (dcoords) {
        // the coordinate gradient rides on the two-pass form's first pass
        if (!two_pass || plan.priv) return cudaErrorInvalidValue;
        if (!plan.staged) return bwd_one<T, D, 1, false, false, true, true>(p, plan, stream);
        switch (plan.nq) {
            case 1: return bwd_one<T, D, 1, true, false, true, true>(p, plan, stream);
            case 4: return bwd_one<T, D, 4, true, false, true, true>(p, plan, stream);
            default: return cudaErrorInvalidValue;
        }
    }
    if (two_pass) {
        if (plan.priv) return cudaErrorInvalidValue;
        if (!plan.staged) return bwd_one<T, D, 1, false, false, true>(p, plan, stream);
        switch (plan.nq) {
            case 1: return bwd_one<T, D, 1, true, false, true>(p, plan, stream);
            case 4: return bwd_one<T, D, 4, true, false, true>(p, plan, stream);
            default: return cudaErrorInvalidValue;
        }
    }
    if (!plan.staged) return bwd_one<T, D, 1, false, false, false>(p, plan, stream);
    if (plan.priv) {
        switch (plan.nq) {
            case 1: return bwd_one<T, D, 1, true, true, false>(p, plan, stream);
            case 4: return bwd_one<T, D, 4, true, true, false>(p, plan, stream);
            default: return cudaErrorInvalidValue;
        }
    }
    switch (plan.nq) {
        case 1: return bwd_one<T, D, 1, true, false, false>(p, plan, stream);
        case 4: return bwd_one<T, D, 4, true, false, false>(p, plan, stream);
        default: return cudaErrorInvalidValue;
    }
}

template <typename T, int D>
inline cudaError_t gather_d(const GatherParams& p, const GatherPlan& plan, cudaStream_t stream) {
    auto kern = bwd_gather_kernel<T, D>;
    static bool done[64] = {};
    cudaError_t e = allow_big_smem(kern, done);
    if (e != cudaSuccess) return e;
    kern<<<(unsigned)plan.gather_ctas, plan.gather_threads, plan.gather_smem, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace detail

}  // namespace dsdpa

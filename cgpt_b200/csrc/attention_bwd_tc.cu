// Tensor-core (tcgen05 / TMEM / TMA) attention backward for sm_100a: 16-bit tensors, head_dim 64 or 128,
// any GQA ratio, causal (with query_position_offset) or full. Three launches, no atomics, no fp32
// gradient scratch, bit-reproducible:
//
//   1. attention_bwd_prep_kernel   delta[b,h,q] = sum_d dO*O and lse2[b,h,q] = LSE * log2(e), both stored
//                                  [batch, heads, seq] so that a tile's 64 or 128 values are contiguous.
//   2. attention_bwd_tc_kernel<MODE_DQ>   one CTA per (128-query tile, query head, batch); streams 64-key
//                                  tiles: S = Q K^T, dP = dO V^T -> dS -> dQ += dS K          (3 MMAs / tile)
//   3. attention_bwd_tc_kernel<MODE_DKV>  one CTA per (128-key tile, kv head, batch); streams 64-query
//                                  tiles of every query head of the group: S^T = K Q^T, dP^T = V dO^T ->
//                                  P^T, dS^T -> dV += P^T dO, dK += dS^T Q                     (4 MMAs / tile)
// Like the reference's tensor-core backward (src/ops/backward/attention_backward.cu:1167-1677) S and dP are
// recomputed in both kernels (7 GEMM-equivalents for the 5 algorithmic ones) in exchange for having exactly
// one writer per output element. Rounding points are the reference's: P and scale*dS are rounded to the
// storage dtype before the second products (:1336-1343, :1567-1586); everything else is fp32.
//
// Both kernels are one template. A "stationary" pair of [128, D] tiles (X1, X2) stays in shared memory,
// a "streaming" pair of [64, D] tiles (Y1, Y2) runs through a 4-stage (D 128) or 6-stage (D 64) TMA ring:
//     T1 = X1 Y1^T, T2 = X2 Y2^T            two 128x64 fp32 tiles in TMEM (triple-buffered where 512 columns allow, else double)
//     threads (one per TMEM lane = stationary row; two warpgroups take alternate tiles) turn T1/T2 into 16-bit tiles
//     U (P^T) and W (dS or dS^T),
//     written back into TMEM over the columns of T1/T2 they were computed from (A operands read from TMEM)
//     acc1 += U Y2, acc2 += W Y1 (dKV)   or   acc1 += W Y1 (dQ)      accumulators stay in TMEM
// The streaming tiles serve twice from the same bytes: as K-major B operands of T1/T2 and as N-major
// ("MN-major") B operands of the accumulating products.
#include <cstdlib>
#include <type_traits>

#include "attention.h"
#include "launch_counter.h"
#include "sm100.cuh"

namespace cgpt {

unsigned int* tc_status_device_ptr();   // gemm.cu

namespace {

using namespace sm100;

constexpr int kRows = 128;   // stationary tile rows = TMEM lanes
constexpr int kCols = 64;    // streaming tile rows = columns of T1/T2
constexpr int kBwdThreads = 320;   // warps 0-7 compute (two warpgroups taking alternate streaming tiles), 8 TMA, 9 MMA
constexpr float kLog2e = 1.4426950408889634f;
constexpr int MODE_DQ = 0, MODE_DKV = 1;

// The streaming-tile ring is as deep as shared memory allows: a tile's TMA load takes about 1.2 us under load, a tile's
// MMAs about half of that, and a stage is only released when the accumulating MMAs of its tile have completed, so three
// stages left the MMA thread waiting on every load. U and W never touch shared memory (they live in TMEM, over T1 / T2).
template <int D> struct BwdSmem {
    static constexpr int kStages = D == 128 ? 4 : 6;
    static constexpr int kChunks = D / 64;
    static constexpr int kXBytes = kChunks * kRows * 128;     // one stationary tile
    static constexpr int kYBytes = kChunks * kCols * 128;     // one streaming tile
    static constexpr int kX1 = 0;
    static constexpr int kX2 = kX1 + kXBytes;
    static constexpr int kY = kX2 + kXBytes;                  // [kStages][Y1 | Y2]
    static constexpr int kStats = kY + kStages * 2 * kYBytes; // [kStages][2][64] fp32
    static constexpr int kBars = kStats + kStages * 2 * kCols * 4;
    static constexpr int kLimit = 232448;                     // the 227 KB a CTA may use
    // room to round the dynamic shared-memory base up to 1024 bytes (the 128B swizzle's atom); the kernel checks at run
    // time that the base needs no more than this and reports through the status word otherwise
    static constexpr int kAlignSlack = kLimit - (kBars + 256) < 1024 ? kLimit - (kBars + 256) : 1024;
    static constexpr int kBytes = kBars + 256 + kAlignSlack;
    static_assert(kAlignSlack >= 0, "attention backward shared memory exceeds the 227 KB a CTA may use");
};

// TMEM columns of one CTA (512 in all): the T1 / T2 buffers of the tiles in flight, then the accumulators. The MMA
// thread issues the T products of a tile kTBufs - 1 tiles ahead of the accumulating products; it can only do so
// while a buffer is free, and a buffer is held from the T products of its tile until the accumulating products
// have consumed the U / W written over it. With two buffers the thread has to wait for the compute warps' result
// of tile it before it may issue T(it + 2), so the warps' whole latency per tile (wake-up, TMEM load, exponentials,
// TMEM store, hand-over) sits in the loop: period = (tensor time + compute latency) / 2. Three buffers, wherever
// 512 columns allow them (every case but dK/dV at head_dim 128, whose two accumulators take 256), take that latency
// out of the loop.
template <int D, int MODE> struct BwdTmem {
    static constexpr int kAccCols = (MODE == 1 ? 2 : 1) * D;
    static constexpr int kTBufs = (512 - kAccCols) >= 3 * 2 * kCols ? 3 : 2;
    static constexpr int kT1 = 0;
    static constexpr int kT2 = kTBufs * kCols;
    static constexpr int kAcc = 2 * kTBufs * kCols;
    static_assert(kAcc + kAccCols <= 512, "TMEM columns");
};

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <typename T> __device__ __forceinline__ std::uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ std::uint32_t pack2<__half>(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<std::uint32_t*>(&h);
}
template <> __device__ __forceinline__ std::uint32_t pack2<__nv_bfloat16>(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<std::uint32_t*>(&h);
}

// delta and lse2 in [batch, heads, seq] order. D/8 lanes own one (b, q, h) row of dO / O (one 16-byte chunk each), so
// a warp covers 32/(D/8) rows per group and kPrepUnroll groups per trip, all of whose loads are issued before the
// first use (memory-bound: 2 * D * 2 bytes per row).
constexpr int kPrepUnroll = 4;

template <typename T, int D>
__global__ void __launch_bounds__(256)
attention_bwd_prep_kernel(float* __restrict__ delta_t, float* __restrict__ lse2_t, const T* __restrict__ dout,
                          const T* __restrict__ out, const float* __restrict__ lse, unsigned rows, int sq, int hq,
                          FastDiv div_hq, FastDiv div_sq) {
    // rows = batch * sq * hq fits 31 bits (a tensor of 2^31 rows of D 16-bit values cannot exist on this device); the row's
    // (batch, query, head) comes from two multiply-shift divisions, and the lane group's width is a compile-time constant
    constexpr int lpr = D / 8;                     // lanes per row (8 or 16)
    constexpr int rows_per_group = 32 / lpr;
    const int lane = threadIdx.x & 31;
    const int sub = lane / lpr, l = lane % lpr;
    const unsigned warp_id = blockIdx.x * 8 + (threadIdx.x >> 5);
    const unsigned warps_total = gridDim.x * 8;
    constexpr unsigned per_trip = rows_per_group * kPrepUnroll;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    for (unsigned base = warp_id * per_trip; base < rows; base += warps_total * per_trip) {
        uint4 a[kPrepUnroll], o[kPrepUnroll];
#pragma unroll
        for (int u = 0; u < kPrepUnroll; ++u) {
            const unsigned row = base + u * rows_per_group + sub;
            const long long off = static_cast<long long>(row) * D + l * 8;
            a[u] = row < rows ? __ldcs(reinterpret_cast<const uint4*>(dout + off)) : zero;
            o[u] = row < rows ? __ldg(reinterpret_cast<const uint4*>(out + off)) : zero;
        }
#pragma unroll
        for (int u = 0; u < kPrepUnroll; ++u) {
            const unsigned row = base + u * rows_per_group + sub;
            Pack<T, 8> pa, po;
            *reinterpret_cast<uint4*>(&pa) = a[u];
            *reinterpret_cast<uint4*>(&po) = o[u];
            float fa[8], fo[8];
            unpack_pack(fa, pa);
            unpack_pack(fo, po);
            float s = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) s = fmaf(fa[e], fo[e], s);
#pragma unroll
            for (int off = lpr >> 1; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
            if (l == 0 && row < rows) {
                unsigned bq, h, b, q;
                div_hq.divmod(row, bq, h);
                div_sq.divmod(bq, b, q);
                const long long t = (static_cast<long long>(b) * hq + h) * sq + q;
                delta_t[t] = s;
                lse2_t[t] = lse[row] * kLog2e;
            }
        }
    }
}

#include "attention_bwd_roles.cuh"
#include "attention_bwd_compute.cuh"
#include "attention_bwd_main.cuh"

}  // namespace

int attention_backward_tc_launch(void* dq, void* dk, void* dv, const void* dout, const void* out, const float* lse,
                                 const void* q, const void* k, const void* v, const AttnDims& dm, int accumulate, int dtype,
                                 cudaStream_t s) {
    if (dtype == CGPT_DTYPE_F32 || (dm.d != 64 && dm.d != 128)) return CGPT_ERR_UNSUPPORTED;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out) || !aligned16(dout) || !aligned16(dq) ||
        !aligned16(dk) || !aligned16(dv))
        return CGPT_ERR_UNSUPPORTED;
    if (static_cast<long long>((dm.sq + kRows - 1) / kRows + (dm.sk + kRows - 1) / kRows) * dm.hq * dm.batch > 0x7fffffffll) return CGPT_ERR_UNSUPPORTED;   // 1-D grids
    if (dtype == CGPT_DTYPE_F16)
        return dm.d == 64 ? launch_backward<__half, 64>(dq, dk, dv, dout, out, lse, q, k, v, dm, accumulate, dtype, s)
                          : launch_backward<__half, 128>(dq, dk, dv, dout, out, lse, q, k, v, dm, accumulate, dtype, s);
    return dm.d == 64 ? launch_backward<__nv_bfloat16, 64>(dq, dk, dv, dout, out, lse, q, k, v, dm, accumulate, dtype, s)
                      : launch_backward<__nv_bfloat16, 128>(dq, dk, dv, dout, out, lse, q, k, v, dm, accumulate, dtype, s);
}

}  // namespace cgpt

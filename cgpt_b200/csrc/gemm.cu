// Dense 16-bit GEMM with fp32 accumulation on the sm_100a tensor cores (tcgen05.mma, accumulator in
// TMEM, operands staged by TMA into 128-byte-swizzled shared memory), plus a plain SIMT kernel for
// fp32 tensors and shapes TMA cannot address.
//
// It serves the three contractions of a linear layer Y = X W^T (reference: src/ops/linear.cu and
// src/ops/backward/linear_backward.cu:135-148, which call cuBLASLt):
//   forward  Y [T,out]  = X [T,in]  * W [out,in]^T     A K-major,  B K-major
//   dX       dX[T,in]   = dY[T,out] * W [out,in]       A K-major,  B N-major (MN-major tile)
//   dW       dW[out,in] = dY[T,out]^T * X [T,in]       A M-major,  B N-major, reduction over T
//
// Kernel shape (gemm_persistent.cuh): one persistent CTA per SM walks 128 x BN tiles (BN = 128 or 256), each for a
// slice of K. Warp 0 issues the TMA loads into a STAGES-deep ring, warp 1 issues tcgen05.mma (128 x BN x 16 per
// instruction, four per 64-wide K block) and commits each stage back to the producer, warps 2-5 drain the fp32
// accumulator from TMEM (tcgen05.ld), convert and store. Split-K writes fp32 partials that a small
// kernel sums in a fixed order (deterministic; used when the tile count alone cannot fill 148 SMs,
// e.g. dW with K = tokens). Algorithmic work: 2*M*N*K flops.
#include <cstdlib>
#include <mutex>
#include <type_traits>
#include <vector>

#include "launch_counter.h"
#include "sm100.cuh"

namespace cgpt {

// ------------------------------------------------------------------------------------ tensor maps
namespace {
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn g_encode = nullptr;
std::once_flag g_encode_once;

void load_encode() {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
        g_encode = reinterpret_cast<EncodeFn>(fn);
}
}  // namespace

int make_tensor_map(CUtensorMap* map, int dtype, const void* base, int rank, const std::uint64_t* dims,
                    const std::uint64_t* strides_bytes, const std::uint32_t* box) {
    std::call_once(g_encode_once, load_encode);
    if (g_encode == nullptr) return CGPT_ERR_UNSUPPORTED;
    cuuint64_t gdim[5], gstride[5];
    cuuint32_t gbox[5], estride[5];
    for (int i = 0; i < rank; ++i) {
        gdim[i] = dims[i];
        gbox[i] = box[i];
        estride[i] = 1;
        if (i + 1 < rank) gstride[i] = strides_bytes[i];
    }
    const CUtensorMapDataType dt = dtype == CGPT_DTYPE_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                 : dtype == CGPT_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                            : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    const CUresult r = g_encode(map, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdim, gstride, gbox,
                                estride, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? CGPT_OK : CGPT_ERR_SHAPE;
}

namespace {

using namespace sm100;

constexpr int BM = 128;
constexpr int BK = 64;          // 64 x 16-bit = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int kGemmThreads = 192;

template <int BN> struct GemmCfg {
    static constexpr int kStages = BN == 256 ? 4 : 6;
    static constexpr int kStoreBufs = 2;   // staging buffers of the TMA-store epilogue
    static constexpr int kABytes = BM * BK * 2;
    static constexpr int kBBytes = BN * BK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/ + kStoreBufs * BM * 128 /*store staging*/;
};

// Device status word shared by the contraction kernels: non-zero means a bounded wait ran out.
__device__ unsigned int g_gemm_status = 0;

enum : int { kEpiStore = 0, kEpiAccumulate = 1, kEpiPartial = 2, kEpiNone = 3, kEpiStoreTma = 4, kEpiStageOnly = 5, kEpiStoreTmaFixed = 6, kEpiStoreTmaResidual = 7,
              kEpiRowTilesFastest = 0x100 /* flag for the pair kernel, or-ed to the mode: order of its work units */ };

// Optional timing of the tensor-core GEMM launches (eager mode only, never during stream capture):
// a CUDA event pair around every tensor-core GEMM launch plus its algorithmic FLOPs.
struct GemmTiming {
    bool enabled = false;
    std::vector<cudaEvent_t> events;   // pairs
    std::vector<double> flops;
    std::size_t used = 0;              // events used
};
GemmTiming g_timing;

// out[m,n] = sum_s partial[s,m,n] (+ old out when accumulate), fixed order.
template <typename T>
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(T* __restrict__ out, const float* __restrict__ partial, long long mn, long long split_stride, int splits,
                     int accumulate) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 4;
    for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < mn; i += stride) {
        if (i + 4 <= mn && (mn & 3) == 0) {
            float4 acc = *reinterpret_cast<const float4*>(partial + i);
            for (int s = 1; s < splits; ++s) {
                const float4 p = *reinterpret_cast<const float4*>(partial + s * split_stride + i);
                acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
            }
            float v[4] = {acc.x, acc.y, acc.z, acc.w};
            if (accumulate) {
                float old[4];
                load_vec<T, 4>(old, out + i);
#pragma unroll
                for (int e = 0; e < 4; ++e) v[e] += old[e];
            }
            store_vec<T, 4>(out + i, v);
        } else {
            for (long long j = i; j < mn && j < i + 4; ++j) {
                float acc = 0.f;
                for (int s = 0; s < splits; ++s) acc += partial[s * split_stride + j];
                if (accumulate) acc += to_f32<T>(out[j]);
                out[j] = from_f32<T>(acc);
            }
        }
    }
}

// The same for up to three outputs whose partial tiles sit one after the other in the partial buffer (the weight gradients
// of projections that share their input, computed by one launch): one reduce launch instead of one per output.
// Every count is a multiple of 4 (host check).
struct ReduceGroups {
    void* out[3];
    long long first[3];    // offset of the group's first element inside one split's partial block
    long long end[3];      // running end of the groups in the concatenated index space
    int groups;
};
template <typename T>
__global__ void __launch_bounds__(256)
splitk_reduce_groups_kernel(ReduceGroups g, const float* __restrict__ partial, long long split_stride, int splits, int accumulate) {
    const long long total = g.end[g.groups - 1];
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 4;
    for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < total; i += stride) {
        int grp = 0;
        long long begin = 0;
        if (g.groups > 1 && i >= g.end[0]) { grp = 1; begin = g.end[0]; }
        if (g.groups > 2 && i >= g.end[1]) { grp = 2; begin = g.end[1]; }
        const long long local = i - begin;
        const float* src = partial + g.first[grp] + local;
        float4 acc = *reinterpret_cast<const float4*>(src);
        for (int s = 1; s < splits; ++s) {
            const float4 p = *reinterpret_cast<const float4*>(src + s * split_stride);
            acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
        }
        float v[4] = {acc.x, acc.y, acc.z, acc.w};
        T* out = static_cast<T*>(g.out[grp]) + local;
        if (accumulate) {
            float old[4];
            load_vec<T, 4>(old, out);
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] += old[e];
        }
        store_vec<T, 4>(out, v);
    }
}

// ------------------------------------------------------------------------------------- SIMT fallback
// C[m,n] (+)= sum_k A(m,k) * B(n,k) with arbitrary element strides; 64x64 tile, 4x4 per thread, fp32.
template <typename T>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(T* __restrict__ C, const T* __restrict__ A, const T* __restrict__ B, int M, int N, int K,
                 long long a_sm, long long a_sk, long long b_sn, long long b_sk, int accumulate) {
    __shared__ float As[16][65];
    __shared__ float Bs[16][65];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += 16) {
        for (int i = threadIdx.x; i < 64 * 16; i += 256) {
            const int kk = i & 15, r = i >> 4;
            const int m = m0 + r, n = n0 + r, k = k0 + kk;
            As[kk][r] = (m < M && k < K) ? to_f32<T>(A[m * a_sm + k * a_sk]) : 0.f;
            Bs[kk][r] = (n < N && k < K) ? to_f32<T>(B[n * b_sn + k * b_sk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { a[i] = As[kk][ty * 4 + i]; b[i] = Bs[kk][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
    for (int i = 0; i < 4; ++i)
        for (int j = 0; j < 4; ++j) {
            const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (m < M && n < N) {
                float v = acc[i][j];
                T* dst = C + static_cast<long long>(m) * N + n;
                if (accumulate) v += to_f32<T>(*dst);
                *dst = from_f32<T>(v);
            }
        }
}

// Column sums of a [rows, cols] matrix (bias gradient), coalesced: each CTA owns 32 columns and
// strides over rows with 8 row lanes; fp32, fixed order.
template <typename T>
__global__ void __launch_bounds__(256)
column_sum_kernel(T* __restrict__ out, const T* __restrict__ in, long long rows, int cols, int accumulate) {
    __shared__ float tile[8][33];
    const int col = blockIdx.x * 32 + (threadIdx.x & 31);
    const int rl = threadIdx.x >> 5;
    float acc = 0.f;
    if (col < cols)
        for (long long r = rl; r < rows; r += 8) acc += to_f32<T>(in[r * cols + col]);
    tile[rl][threadIdx.x & 31] = acc;
    __syncthreads();
    if (rl == 0 && col < cols) {
        float total = 0.f;
#pragma unroll
        for (int r = 0; r < 8; ++r) total += tile[r][threadIdx.x & 31];
        if (accumulate) total += to_f32<T>(out[col]);
        out[col] = from_f32<T>(total);
    }
}

#include "gemm_persistent.cuh"
#include "gemm_pair.cuh"
#include "gemm_swiglu.cuh"

// C[M,N] (+)= sum_i A_i[M,K_i] * B_i, i < segments (1..kMaxKSegments): one launch, one pass over C.
// Whether the CTA-pair kernel (gemm_pair.cuh) is used where its tile shape applies. Diagnosis builds can switch it off
// (CGPT_B200_GEMM_PAIR=0) to compare the two kernels.
inline bool pair_kernel_enabled() {
    static const bool on = [] { const char* e = diagnosis_env("CGPT_B200_GEMM_PAIR"); return !(e != nullptr && e[0] == '0'); }();
    return on;
}

// PAIR: 256 x 256 tiles on CTA pairs (BN must be 256) instead of 128 x BN tiles on single CTAs.
template <typename T, int BN, bool A_MN, bool B_MN, bool PAIR = false>
int launch_tc(T* C, const T* const* As, const T* const* Bs, const int* Ks, int segments, int M, int N, int accumulate, int dtype,
              cudaStream_t s, const T* residual = nullptr) {
    using Cfg = GemmCfg<BN>;
    static_assert(!PAIR || BN == kPairBN, "the pair kernel has 256-column tiles");
    constexpr int kTileM = PAIR ? kPairBM : BM;        // rows of a work unit's tile
    constexpr int kBoxN = PAIR ? BN / 2 : BN;          // B rows (columns of C) one CTA loads per K block
    // a residual operand is added only by the pair kernel's TMA-store epilogue
    if (residual != nullptr && (!PAIR || accumulate || N % 64 != 0 || !aligned16(C) || !aligned16(residual))) return CGPT_ERR_UNSUPPORTED;
    GemmOperands ops;
    ops.segments = segments;
    ops.groups = 1;
    ops.group_dim = 0;
    ops.tile_end[0] = ops.tile_end[1] = ops.tile_end[2] = 0;
    int total_kb = 0;
    long long K = 0;   // summed: split heuristics and the FLOP count
    for (int i = 0; i < kMaxKSegments; ++i) {
        const int g = i < segments ? i : 0;   // unused slots repeat segment 0 so that every map is valid
        const int Ki = Ks[g];
        // innermost dimension first
        const std::uint64_t a_dims_k[2] = {static_cast<std::uint64_t>(Ki), static_cast<std::uint64_t>(M)};
        const std::uint64_t a_dims_m[2] = {static_cast<std::uint64_t>(M), static_cast<std::uint64_t>(Ki)};
        const std::uint64_t a_st_k[1] = {static_cast<std::uint64_t>(Ki) * 2}, a_st_m[1] = {static_cast<std::uint64_t>(M) * 2};
        const std::uint32_t a_box_k[2] = {BK, BM}, a_box_m[2] = {64, BK};
        CGPT_TRY(make_tensor_map(&ops.a[i], dtype, As[g], 2, A_MN ? a_dims_m : a_dims_k, A_MN ? a_st_m : a_st_k, A_MN ? a_box_m : a_box_k));
        const std::uint64_t b_dims_k[2] = {static_cast<std::uint64_t>(Ki), static_cast<std::uint64_t>(N)};
        const std::uint64_t b_dims_n[2] = {static_cast<std::uint64_t>(N), static_cast<std::uint64_t>(Ki)};
        const std::uint64_t b_st_k[1] = {static_cast<std::uint64_t>(Ki) * 2}, b_st_n[1] = {static_cast<std::uint64_t>(N) * 2};
        const std::uint32_t b_box_k[2] = {BK, kBoxN}, b_box_n[2] = {64, BK};
        CGPT_TRY(make_tensor_map(&ops.b[i], dtype, Bs[g], 2, B_MN ? b_dims_n : b_dims_k, B_MN ? b_st_n : b_st_k, B_MN ? b_box_n : b_box_k));
        if (i < segments) {
            total_kb += (Ki + BK - 1) / BK;
            K += Ki;
        }
        ops.kb_end[i] = total_kb;
    }
    const CUtensorMap& ta = ops.a[0];
    const int tiles_m = (M + kTileM - 1) / kTileM, tiles_n = (N + BN - 1) / BN;
    // Split K when the output tiles alone leave most SMs (pairs) idle and K is long enough to amortise it.
    constexpr int kWorkers = PAIR ? kNumSMs / 2 : kNumSMs;
    int splits = 1;
    const int tiles = tiles_m * tiles_n;
    if (tiles < kWorkers) {
        splits = kWorkers / tiles;
        const int max_by_k = total_kb / 8 > 0 ? total_kb / 8 : 1;   // at least 8 K blocks (512) per split
        if (splits > max_by_k) splits = max_by_k;
        if (splits > 32) splits = 32;
        if (splits < 1) splits = 1;
    }
    int kb_per_split = (total_kb + splits - 1) / splits;
    splits = (total_kb + kb_per_split - 1) / kb_per_split;   // no empty split
    float* partial = nullptr;
    if (splits > 1 && residual != nullptr) return CGPT_ERR_UNSUPPORTED;
    if (splits > 1) {
        void* scratch = nullptr;
        CGPT_TRY(scratch_get(&scratch, static_cast<std::size_t>(splits) * M * N * sizeof(float), s));
        partial = static_cast<float*>(scratch);
    }
    void (*pkernel)(GemmOperands, GemmOutputs, T*, float*, int, int, int, int, int, int, int, int) = nullptr;
    int smem_bytes = Cfg::kSmemBytes;
    if constexpr (PAIR) {
        pkernel = gemm_tcgen05_pair_kernel<T, A_MN, B_MN>;
        smem_bytes = PairCfg::kSmemBytes;
    } else {
        pkernel = gemm_tcgen05_persistent_kernel<T, BN, A_MN, B_MN>;
    }
    static PerDeviceOnce attr_once;
    if (attr_once.needed()) {
        CGPT_CUDA_TRY(cudaFuncSetAttribute(pkernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
        attr_once.done();
    }
    int epi = splits > 1 ? kEpiPartial : (accumulate ? kEpiAccumulate : kEpiStore);
    {   // diagnosis builds only: CGPT_B200_GEMM_NOSTORE=1 drains the accumulator but skips the global stores
        static const int nostore = [] { const char* e = diagnosis_env("CGPT_B200_GEMM_NOSTORE"); return e ? std::atoi(e) : 0; }();
        if (nostore == 1) epi = kEpiNone;
    }
    const bool timed = g_timing.enabled && g_timing.used + 2 <= g_timing.events.size();
    if (timed) CGPT_CUDA_TRY(cudaEventRecord(g_timing.events[g_timing.used], s));
    {
        const long long units = static_cast<long long>(tiles) * splits;
        unsigned grid = static_cast<unsigned>(units < kNumSMs ? units : kNumSMs);
        if (PAIR) {
            grid = static_cast<unsigned>(pair_grid(reinterpret_cast<const void*>(pkernel), static_cast<int>(units < kNumSMs ? units : kNumSMs)));
            if (grid == 0) return CGPT_ERR_UNSUPPORTED;   // clusters of 2 cannot be scheduled here: the caller takes the single-CTA kernel
        }
        // Plain stores of 16-bit output go through shared memory and TMA (needs a 16-byte aligned C and N % 8 == 0).
        GemmOutputs outs;
        outs.c[0] = outs.c[1] = outs.c[2] = ta;      // placeholders: only read by the TMA-store epilogue
        CUtensorMap& tc = outs.c[0];
        if (epi == kEpiStore && aligned16(C) && N % 8 == 0) {
            const std::uint64_t dims_c[2] = {static_cast<std::uint64_t>(N), static_cast<std::uint64_t>(M)};
            const std::uint64_t st_c[1] = {static_cast<std::uint64_t>(N) * 2};
            const std::uint32_t box_c[2] = {64, BM};
            CGPT_TRY(make_tensor_map(&tc, dtype, C, 2, dims_c, st_c, box_c));
            epi = kEpiStoreTma;
            if (PAIR && residual != nullptr) epi = kEpiStoreTmaResidual;
            // diagnosis builds only: CGPT_B200_GEMM_NOSTORE=2 stages the tile in shared memory but never issues the TMA store
            // and =3 issues every TMA store to the first 16 KB of C (same store mechanics, no memory-system load)
            static const int diag = [] { const char* e = diagnosis_env("CGPT_B200_GEMM_NOSTORE"); return e ? std::atoi(e) : 0; }();
            if (!PAIR && diag == 2) epi = kEpiStageOnly;
            if (!PAIR && diag == 3) epi = kEpiStoreTmaFixed;
        }
        outs.c[1] = outs.c[2] = outs.c[0];
        T* c_arg = epi == kEpiStoreTmaResidual ? const_cast<T*>(residual) : C;    // that epilogue reads it, the store goes through the map
        // B larger than A and larger than a fraction of L2 (an LM-head-shaped product): walk the row tiles first
        if (PAIR && splits == 1 && static_cast<long long>(N) > static_cast<long long>(M) && static_cast<long long>(N) * K * 2 > (32ll << 20))
            epi |= kEpiRowTilesFastest;
        pkernel<<<grid, kGemmThreads, smem_bytes, s>>>(ops, outs, c_arg, partial, M, N, total_kb, tiles_m, tiles_n, splits, kb_per_split, epi);
    }
    count_launch();
    CGPT_LAUNCH_CHECK();
    if (timed) {
        CGPT_CUDA_TRY(cudaEventRecord(g_timing.events[g_timing.used + 1], s));
        g_timing.used += 2;
        g_timing.flops.push_back(2.0 * M * N * K);
    }
    if (splits > 1) {
        const long long mn = static_cast<long long>(M) * N;
        long long blocks = (mn / 4 + 255) / 256;
        if (blocks > kNumSMs * 8) blocks = kNumSMs * 8;
        if (blocks < 1) blocks = 1;
        splitk_reduce_kernel<T><<<static_cast<unsigned>(blocks), 256, 0, s>>>(C, partial, mn, mn, splits, accumulate);
        count_launch();
        CGPT_LAUNCH_CHECK();
    }
    return CGPT_OK;
}

template <typename T>
int launch_tc_layout(T* C, const T* const* A, const T* const* B, const int* K, int segments, int M, int N, int a_mn, int b_mn,
                     int accumulate, int dtype, cudaStream_t s, const T* residual = nullptr) {
    // 128x256 tiles whenever N allows: a 128x128 tile needs as many shared-memory operand bytes per MMA as the
    // tensor core can consume, 128x256 needs 3/4 of that per FLOP. Few tiles are compensated by split-K.
    const bool wide = N >= 256;
    // 256 x 256 tiles on CTA pairs when both dimensions allow them (two thirds of the shared-memory traffic per FLOP)
    // Measured on the training shapes: +1..4 % on the forward and dX products, +11 % on the LM-head logits, but -15 % on
    // the weight-gradient products (both operands MN-major, K = tokens, split-K), which therefore stay on single CTAs.
    const bool pair = wide && M >= kPairBM && a_mn == 0 && pair_kernel_enabled();
#define CGPT_GEMM_CASE(AM, BMN)                                                                  \
    if (a_mn == AM && b_mn == BMN) {                                                             \
        if (pair) {                                                                              \
            const int rc = launch_tc<T, 256, AM != 0, BMN != 0, true>(C, A, B, K, segments, M, N, accumulate, dtype, s, residual); \
            if (rc != CGPT_ERR_UNSUPPORTED) return rc;                                           \
        }                                                                                        \
        if (residual != nullptr) return CGPT_ERR_UNSUPPORTED;                                    \
        return wide ? launch_tc<T, 256, AM != 0, BMN != 0>(C, A, B, K, segments, M, N, accumulate, dtype, s) \
                    : launch_tc<T, 128, AM != 0, BMN != 0>(C, A, B, K, segments, M, N, accumulate, dtype, s); \
    }
    CGPT_GEMM_CASE(0, 0)
    CGPT_GEMM_CASE(0, 1)
    CGPT_GEMM_CASE(1, 1)
    CGPT_GEMM_CASE(1, 0)
#undef CGPT_GEMM_CASE
    return CGPT_ERR_OPTION;
}

// Y_g[M, N_g] = A[M, K] * B_g[N_g, K]^T for up to three outputs that share A, as ONE launch: the N tiles of all groups
// form one work list (better wave quantisation than three launches, A read through L2 by neighbouring CTAs).
// Tensor-core path only (16-bit, aligned, N_g % 8 == 0); returns CGPT_ERR_UNSUPPORTED otherwise.
template <typename T, bool PAIR = false>
int launch_tc_groups(T* const* Cs, const T* A, const T* const* Bs, const int* Ns, int groups, int M, int K, int dtype, cudaStream_t s) {
    constexpr int BN = 256;
    using Cfg = GemmCfg<BN>;
    constexpr int kTileM = PAIR ? kPairBM : BM;
    constexpr int kWorkers = PAIR ? kNumSMs / 2 : kNumSMs;
    if (groups < 1 || groups > kMaxKSegments || !aligned16(A) || K % 8 != 0 || K < 32) return CGPT_ERR_UNSUPPORTED;
    if (PAIR && M < kPairBM) return CGPT_ERR_UNSUPPORTED;
    GemmOperands ops;
    GemmOutputs outs;
    ops.segments = 1;
    ops.groups = groups;
    ops.group_dim = 0;
    const std::uint64_t a_dims[2] = {static_cast<std::uint64_t>(K), static_cast<std::uint64_t>(M)};
    const std::uint64_t k_st[1] = {static_cast<std::uint64_t>(K) * 2};
    const std::uint32_t a_box[2] = {BK, BM}, b_box[2] = {BK, PAIR ? BN / 2 : BN}, c_box[2] = {64, BM};
    int tiles_n = 0;
    double flops = 0.0;
    for (int i = 0; i < kMaxKSegments; ++i) {
        const int g = i < groups ? i : 0;
        if (!aligned16(Cs[g]) || !aligned16(Bs[g]) || Ns[g] % 8 != 0 || Ns[g] <= 0) return CGPT_ERR_UNSUPPORTED;
        CGPT_TRY(make_tensor_map(&ops.a[i], dtype, A, 2, a_dims, k_st, a_box));
        const std::uint64_t b_dims[2] = {static_cast<std::uint64_t>(K), static_cast<std::uint64_t>(Ns[g])};
        CGPT_TRY(make_tensor_map(&ops.b[i], dtype, Bs[g], 2, b_dims, k_st, b_box));
        const std::uint64_t c_dims[2] = {static_cast<std::uint64_t>(Ns[g]), static_cast<std::uint64_t>(M)};
        const std::uint64_t c_st[1] = {static_cast<std::uint64_t>(Ns[g]) * 2};
        CGPT_TRY(make_tensor_map(&outs.c[i], dtype, Cs[g], 2, c_dims, c_st, c_box));
        if (i < groups) {
            tiles_n += (Ns[g] + BN - 1) / BN;
            flops += 2.0 * M * Ns[g] * K;
        }
        ops.tile_end[i] = tiles_n;
        ops.kb_end[i] = (K + BK - 1) / BK;
    }
    const int tiles_m = (M + kTileM - 1) / kTileM;
    const long long units = static_cast<long long>(tiles_m) * tiles_n;
    if (units < kWorkers) return CGPT_ERR_UNSUPPORTED;   // too small to be worth it: no split-K in this form
    void (*pkernel)(GemmOperands, GemmOutputs, T*, float*, int, int, int, int, int, int, int, int) = nullptr;
    int smem_bytes = Cfg::kSmemBytes;
    unsigned grid = kNumSMs;
    if constexpr (PAIR) {
        pkernel = gemm_tcgen05_pair_kernel<T, false, false>;
        smem_bytes = PairCfg::kSmemBytes;
    } else {
        pkernel = gemm_tcgen05_persistent_kernel<T, BN, false, false>;
    }
    static PerDeviceOnce attr_once;
    if (attr_once.needed()) {
        CGPT_CUDA_TRY(cudaFuncSetAttribute(pkernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
        attr_once.done();
    }
    if (PAIR) {
        grid = static_cast<unsigned>(pair_grid(reinterpret_cast<const void*>(pkernel), kNumSMs));
        if (grid == 0) return CGPT_ERR_UNSUPPORTED;
    }
    const bool timed = g_timing.enabled && g_timing.used + 2 <= g_timing.events.size();
    if (timed) CGPT_CUDA_TRY(cudaEventRecord(g_timing.events[g_timing.used], s));
    pkernel<<<grid, kGemmThreads, smem_bytes, s>>>(ops, outs, Cs[0], nullptr, M, Ns[0], (K + BK - 1) / BK, tiles_m, tiles_n, 1,
                                                  (K + BK - 1) / BK, kEpiStoreTma);
    count_launch();
    CGPT_LAUNCH_CHECK();
    if (timed) {
        CGPT_CUDA_TRY(cudaEventRecord(g_timing.events[g_timing.used + 1], s));
        g_timing.used += 2;
        g_timing.flops.push_back(flops);
    }
    return CGPT_OK;
}

// dW_g[M_g, N] (+)= dY_g[K, M_g]^T X[K, N] for up to three weight gradients that share X, as ONE launch: the M tiles of
// all groups form one work list (both operands MN-major, K = tokens). With few tiles K is split as in the plain
// launcher: fp32 partials [split][sum of padded M_g][N], then one fixed-order reduce per group.
template <typename T>
int launch_tc_mgroups(T* const* Cs, const T* const* As, const T* B, const int* Ms, int groups, int N, int K, int accumulate,
                      int dtype, cudaStream_t s) {
    constexpr int BN = 256;
    using Cfg = GemmCfg<BN>;
    constexpr int kTileM = BM;
    constexpr int kWorkers = kNumSMs;
    if (groups < 1 || groups > kMaxKSegments || !aligned16(B) || N % 8 != 0 || N < BN || K < 32) return CGPT_ERR_UNSUPPORTED;
    GemmOperands ops;
    GemmOutputs outs;
    ops.segments = 1;
    ops.groups = groups;
    ops.group_dim = 1;
    const std::uint64_t b_dims[2] = {static_cast<std::uint64_t>(N), static_cast<std::uint64_t>(K)};
    const std::uint64_t b_st[1] = {static_cast<std::uint64_t>(N) * 2};
    const std::uint32_t mn_box[2] = {64, BK}, c_box[2] = {64, BM};
    int tiles_m = 0;
    double flops = 0.0;
    int m_first[kMaxKSegments] = {0, 0, 0};
    for (int i = 0; i < kMaxKSegments; ++i) {
        const int g = i < groups ? i : 0;
        if (!aligned16(Cs[g]) || !aligned16(As[g]) || Ms[g] % 8 != 0 || Ms[g] <= 0) return CGPT_ERR_UNSUPPORTED;
        const std::uint64_t a_dims[2] = {static_cast<std::uint64_t>(Ms[g]), static_cast<std::uint64_t>(K)};
        const std::uint64_t a_st[1] = {static_cast<std::uint64_t>(Ms[g]) * 2};
        CGPT_TRY(make_tensor_map(&ops.a[i], dtype, As[g], 2, a_dims, a_st, mn_box));
        CGPT_TRY(make_tensor_map(&ops.b[i], dtype, B, 2, b_dims, b_st, mn_box));
        const std::uint64_t c_dims[2] = {static_cast<std::uint64_t>(N), static_cast<std::uint64_t>(Ms[g])};
        CGPT_TRY(make_tensor_map(&outs.c[i], dtype, Cs[g], 2, c_dims, b_st, c_box));
        if (i < groups) {
            m_first[i] = tiles_m * kTileM;
            tiles_m += (Ms[g] + kTileM - 1) / kTileM;
            flops += 2.0 * Ms[g] * N * K;
        }
        ops.tile_end[i] = tiles_m;
        ops.kb_end[i] = (K + BK - 1) / BK;
    }
    const int tiles_n = (N + BN - 1) / BN;
    const int total_kb = (K + BK - 1) / BK;
    const int tiles = tiles_m * tiles_n;
    int splits = 1;
    if (tiles < kWorkers) {
        splits = kWorkers / tiles;
        const int max_by_k = total_kb / 8 > 0 ? total_kb / 8 : 1;
        if (splits > max_by_k) splits = max_by_k;
        if (splits > 32) splits = 32;
        if (splits < 1) splits = 1;
    }
    if (accumulate && splits == 1) splits = total_kb >= 2 ? 2 : 1;   // the read-add-store of dW happens in the reduce kernel
    if (accumulate && splits == 1) return CGPT_ERR_UNSUPPORTED;
    const int kb_per_split = (total_kb + splits - 1) / splits;
    splits = (total_kb + kb_per_split - 1) / kb_per_split;
    const int m_pad = tiles_m * kTileM;
    float* partial = nullptr;
    if (splits > 1) {
        void* scratch = nullptr;
        CGPT_TRY(scratch_get(&scratch, static_cast<std::size_t>(splits) * m_pad * N * sizeof(float), s));
        partial = static_cast<float*>(scratch);
    }
    // single-CTA tiles: the CTA-pair kernel measured 15 % slower on these products (both operands MN-major, split-K)
    auto* pkernel = gemm_tcgen05_persistent_kernel<T, BN, true, true>;
    const int smem_bytes = Cfg::kSmemBytes;
    static PerDeviceOnce attr_once;
    if (attr_once.needed()) {
        CGPT_CUDA_TRY(cudaFuncSetAttribute(pkernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
        attr_once.done();
    }
    const long long units = static_cast<long long>(tiles) * splits;
    const unsigned grid = static_cast<unsigned>(units < kNumSMs ? units : kNumSMs);
    const bool timed = g_timing.enabled && g_timing.used + 2 <= g_timing.events.size();
    if (timed) CGPT_CUDA_TRY(cudaEventRecord(g_timing.events[g_timing.used], s));
    pkernel<<<grid, kGemmThreads, smem_bytes, s>>>(ops, outs, Cs[0], partial, m_pad, N, total_kb, tiles_m, tiles_n, splits,
                                                  kb_per_split, splits > 1 ? kEpiPartial : kEpiStoreTma);
    count_launch();
    CGPT_LAUNCH_CHECK();
    if (timed) {
        CGPT_CUDA_TRY(cudaEventRecord(g_timing.events[g_timing.used + 1], s));
        g_timing.used += 2;
        g_timing.flops.push_back(flops);
    }
    if (splits > 1) {   // one reduce launch for all groups (every M_g * N is a multiple of 4: M_g % 8 == 0)
        const long long split_stride = static_cast<long long>(m_pad) * N;
        ReduceGroups rg;
        rg.groups = groups;
        long long total = 0;
        for (int g = 0; g < 3; ++g) {
            const int gg = g < groups ? g : 0;
            rg.out[g] = Cs[gg];
            rg.first[g] = static_cast<long long>(m_first[gg]) * N;
            if (g < groups) total += static_cast<long long>(Ms[g]) * N;
            rg.end[g] = total;
        }
        long long blocks = (total / 4 + 255) / 256;
        const long long cap = static_cast<long long>(kNumSMs) *
                              resident_ctas_per_sm(reinterpret_cast<const void*>(splitk_reduce_groups_kernel<T>), 256, 0);
        if (blocks > cap) blocks = cap;
        if (blocks < 1) blocks = 1;
        splitk_reduce_groups_kernel<T><<<static_cast<unsigned>(blocks), 256, 0, s>>>(rg, partial, split_stride, splits, accumulate);
        count_launch();
        CGPT_LAUNCH_CHECK();
    }
    return CGPT_OK;
}

// LM-head logits X [M,K] * Cw [N,K]^T on CTA pairs with a softmax epilogue (gemm_pair.cuh). out: the logits
// (kSoftmaxStatsStore) or the gradient (kSoftmaxGrad), [M,N]; not used by kSoftmaxStats. No split-K.
template <typename T, int SOFTMAX>
int launch_pair_softmax(T* out, const T* X, const T* Cw, int M, int N, int K, const SoftmaxEpilogue& sx, int dtype, cudaStream_t s) {
    constexpr int BN = kPairBN;
    GemmOperands ops;
    GemmOutputs outs;
    ops.segments = 1;
    ops.groups = 1;
    ops.group_dim = 0;
    const int total_kb = (K + BK - 1) / BK;
    const std::uint64_t a_dims[2] = {static_cast<std::uint64_t>(K), static_cast<std::uint64_t>(M)};
    const std::uint64_t b_dims[2] = {static_cast<std::uint64_t>(K), static_cast<std::uint64_t>(N)};
    const std::uint64_t k_st[1] = {static_cast<std::uint64_t>(K) * 2};
    const std::uint32_t a_box[2] = {BK, BM}, b_box[2] = {BK, BN / 2}, c_box[2] = {64, BM};
    for (int i = 0; i < kMaxKSegments; ++i) {
        CGPT_TRY(make_tensor_map(&ops.a[i], dtype, X, 2, a_dims, k_st, a_box));
        CGPT_TRY(make_tensor_map(&ops.b[i], dtype, Cw, 2, b_dims, k_st, b_box));
        ops.kb_end[i] = total_kb;
        ops.tile_end[i] = 0;
        outs.c[i] = ops.a[0];      // placeholder unless the epilogue stores
    }
    if (SOFTMAX != kSoftmaxStats) {
        const std::uint64_t c_dims[2] = {static_cast<std::uint64_t>(N), static_cast<std::uint64_t>(M)};
        const std::uint64_t c_st[1] = {static_cast<std::uint64_t>(N) * 2};
        CGPT_TRY(make_tensor_map(&outs.c[0], dtype, out, 2, c_dims, c_st, c_box));
        outs.c[1] = outs.c[2] = outs.c[0];
    }
    const int tiles_m = (M + kPairBM - 1) / kPairBM, tiles_n = (N + BN - 1) / BN;
    const long long units = static_cast<long long>(tiles_m) * tiles_n;
    auto* pkernel = gemm_pair_softmax_kernel<T, SOFTMAX>;
    static PerDeviceOnce attr_once;
    if (attr_once.needed()) {
        CGPT_CUDA_TRY(cudaFuncSetAttribute(pkernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PairCfg::kSmemBytes));
        attr_once.done();
    }
    const unsigned grid = static_cast<unsigned>(pair_grid(reinterpret_cast<const void*>(pkernel), static_cast<int>(units < kNumSMs ? units : kNumSMs)));
    if (grid == 0) return CGPT_ERR_UNSUPPORTED;
    const bool timed = g_timing.enabled && g_timing.used + 2 <= g_timing.events.size();
    if (timed) CGPT_CUDA_TRY(cudaEventRecord(g_timing.events[g_timing.used], s));
    pkernel<<<grid, kGemmThreads, PairCfg::kSmemBytes, s>>>(ops, outs, M, N, total_kb, tiles_m, tiles_n, sx);
    count_launch();
    CGPT_LAUNCH_CHECK();
    if (timed) {
        CGPT_CUDA_TRY(cudaEventRecord(g_timing.events[g_timing.used + 1], s));
        g_timing.used += 2;
        g_timing.flops.push_back(2.0 * M * N * K);
    }
    return CGPT_OK;
}

}  // namespace

int gemm_logits_softmax(int mode, void* out, const void* x, const void* c, long long M, long long N, long long K,
                        float2* partial, float* target_logit, const std::uint32_t* targets, const float2* row_stats,
                        float out_scale, int dtype, cudaStream_t s) {
    if (!x || !c || !targets) return CGPT_ERR_NULL;
    if (mode != kSoftmaxStats && !out) return CGPT_ERR_NULL;
    if (mode == kSoftmaxGrad ? !row_stats : (!partial || !target_logit)) return CGPT_ERR_NULL;
    if (dtype != CGPT_DTYPE_F16 && dtype != CGPT_DTYPE_BF16) return CGPT_ERR_UNSUPPORTED;
    if (M < kPairBM || N < kPairBN || K < 32 || M > 0x7fffffffll || N > 0x7fffffffll || K > 0x7fffffffll || K % 8 != 0 || N % 8 != 0 ||
        !aligned16(x) || !aligned16(c) || (out != nullptr && !aligned16(out)) || !pair_kernel_enabled())
        return CGPT_ERR_UNSUPPORTED;
    const SoftmaxEpilogue sx{partial, target_logit, targets, row_stats, out_scale};
    const int m = static_cast<int>(M), n = static_cast<int>(N), k = static_cast<int>(K);
#define CGPT_SOFTMAX_CASE(MODE)                                                                                              \
    if (mode == MODE) {                                                                                                      \
        if (dtype == CGPT_DTYPE_F16)                                                                                         \
            return launch_pair_softmax<__half, MODE>(static_cast<__half*>(out), static_cast<const __half*>(x),              \
                                                     static_cast<const __half*>(c), m, n, k, sx, dtype, s);                  \
        return launch_pair_softmax<__nv_bfloat16, MODE>(static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(x), \
                                                        static_cast<const __nv_bfloat16*>(c), m, n, k, sx, dtype, s);         \
    }
    CGPT_SOFTMAX_CASE(kSoftmaxStatsStore)
    CGPT_SOFTMAX_CASE(kSoftmaxStats)
    CGPT_SOFTMAX_CASE(kSoftmaxGrad)
#undef CGPT_SOFTMAX_CASE
    return CGPT_ERR_OPTION;
}

// C[M,N] (+)= sum_i A_i * B_i over `segments` operand pairs chained along K (1 for a plain GEMM).
// a_mn = 0: A_i stored [M,K_i] (K contiguous); 1: A_i stored [K_i,M]. b_mn = 0: B_i stored [N,K_i]; 1: B_i stored
// [K_i,N]. Chooses the tensor-core kernel for 16-bit dtypes when TMA can address the operands (16-byte aligned
// bases, leading dimensions a multiple of 8 elements), else one SIMT launch per segment.
int gemm_dispatch_segments(void* C, const void* const* A, const void* const* B, const long long* K, int segments, long long M,
                           long long N, int a_mn, int b_mn, int accumulate, int dtype, bool force_simt, cudaStream_t s,
                           const void* residual = nullptr) {
    if (!C || !A || !B || !K) return CGPT_ERR_NULL;
    if (segments < 1 || segments > kMaxKSegments) return CGPT_ERR_SHAPE;
    if (!valid_float_dtype(dtype)) return CGPT_ERR_DTYPE;
    if (M <= 0 || N <= 0 || M > 0x7fffffffll || N > 0x7fffffffll) return CGPT_ERR_SHAPE;
    bool tc_ok = !force_simt && dtype != CGPT_DTYPE_F32 && (reinterpret_cast<std::uintptr_t>(C) % 2 == 0) && M * N >= 64 * 64;
    long long k_total = 0;
    int k32[kMaxKSegments] = {0, 0, 0};
    for (int i = 0; i < segments; ++i) {
        if (!A[i] || !B[i]) return CGPT_ERR_NULL;
        if (K[i] <= 0 || K[i] > 0x7fffffffll) return CGPT_ERR_SHAPE;
        const long long a_ld = a_mn ? M : K[i], b_ld = b_mn ? N : K[i];
        tc_ok = tc_ok && aligned16(A[i]) && aligned16(B[i]) && a_ld % 8 == 0 && b_ld % 8 == 0;
        k_total += K[i];
        k32[i] = static_cast<int>(K[i]);
    }
    if (k_total > 0x7fffffffll) return CGPT_ERR_SHAPE;
    tc_ok = tc_ok && k_total >= 32;
    if (tc_ok) {
        if (dtype == CGPT_DTYPE_F16)
            return launch_tc_layout<__half>(static_cast<__half*>(C), reinterpret_cast<const __half* const*>(A),
                                            reinterpret_cast<const __half* const*>(B), k32, segments, static_cast<int>(M),
                                            static_cast<int>(N), a_mn, b_mn, accumulate, dtype, s, static_cast<const __half*>(residual));
        return launch_tc_layout<__nv_bfloat16>(static_cast<__nv_bfloat16*>(C), reinterpret_cast<const __nv_bfloat16* const*>(A),
                                               reinterpret_cast<const __nv_bfloat16* const*>(B), k32, segments, static_cast<int>(M),
                                               static_cast<int>(N), a_mn, b_mn, accumulate, dtype, s,
                                               static_cast<const __nv_bfloat16*>(residual));
    }
    if (residual != nullptr) return CGPT_ERR_UNSUPPORTED;   // the caller adds it with a separate pass
    for (int i = 0; i < segments; ++i) {
        const long long Ki = K[i];
        const long long a_sm = a_mn ? 1 : Ki, a_sk = a_mn ? M : 1, b_sn = b_mn ? 1 : Ki, b_sk = b_mn ? N : 1;
        const dim3 grid(static_cast<unsigned>((N + 63) / 64), static_cast<unsigned>((M + 63) / 64));
        const int acc = (accumulate || i > 0) ? 1 : 0;
        CGPT_DISPATCH_DTYPE(dtype, T, {
            gemm_simt_kernel<T><<<grid, 256, 0, s>>>(static_cast<T*>(C), static_cast<const T*>(A[i]), static_cast<const T*>(B[i]),
                                                     static_cast<int>(M), static_cast<int>(N), static_cast<int>(Ki), a_sm, a_sk, b_sn,
                                                     b_sk, acc);
            count_launch();
            CGPT_LAUNCH_CHECK();
        });
    }
    return CGPT_OK;
}

int gemm_dispatch(void* C, const void* A, const void* B, long long M, long long N, long long K, int a_mn, int b_mn,
                  int accumulate, int dtype, bool force_simt, cudaStream_t s) {
    if (!C || !A || !B) return CGPT_ERR_NULL;
    if (K <= 0 || K > 0x7fffffffll) return CGPT_ERR_SHAPE;
    if (!force_simt && K < 32) force_simt = true;
    return gemm_dispatch_segments(C, &A, &B, &K, 1, M, N, a_mn, b_mn, accumulate, dtype, force_simt, s);
}

// gate = X Wg^T, up = X Wu^T, act = swiglu(gate, up) in one launch when the tensor-core path applies.
int linear_swiglu_dispatch(void* gate, void* up, void* act, const void* x, const void* wg, const void* wu, long long M, long long N,
                           long long K, int dtype, cudaStream_t s) {
    if (!gate || !up || !act || !x || !wg || !wu) return CGPT_ERR_NULL;
    if (!valid_float_dtype(dtype)) return CGPT_ERR_DTYPE;
    if (M <= 0 || N <= 0 || K <= 0 || M > 0x7fffffffll || N > 0x7fffffffll || K > 0x7fffffffll) return CGPT_ERR_SHAPE;
    int rc = CGPT_ERR_UNSUPPORTED;
    if (dtype == CGPT_DTYPE_F16)
        rc = launch_gemm_swiglu<__half>(static_cast<__half*>(gate), static_cast<__half*>(up), static_cast<__half*>(act),
                                        static_cast<const __half*>(x), static_cast<const __half*>(wg), static_cast<const __half*>(wu),
                                        static_cast<int>(M), static_cast<int>(N), static_cast<int>(K), dtype, s);
    else if (dtype == CGPT_DTYPE_BF16)
        rc = launch_gemm_swiglu<__nv_bfloat16>(static_cast<__nv_bfloat16*>(gate), static_cast<__nv_bfloat16*>(up),
                                               static_cast<__nv_bfloat16*>(act), static_cast<const __nv_bfloat16*>(x),
                                               static_cast<const __nv_bfloat16*>(wg), static_cast<const __nv_bfloat16*>(wu),
                                               static_cast<int>(M), static_cast<int>(N), static_cast<int>(K), dtype, s);
    if (rc != CGPT_ERR_UNSUPPORTED) return rc;
    CGPT_TRY(gemm_dispatch(gate, x, wg, M, N, K, 0, 0, 0, dtype, false, s));
    CGPT_TRY(gemm_dispatch(up, x, wu, M, N, K, 0, 0, 0, dtype, false, s));
    return cgpt_swiglu_forward(act, gate, up, static_cast<size_t>(M) * static_cast<size_t>(N), dtype, s);
}

unsigned int* tc_status_device_ptr() {
    static unsigned int* ptrs[64] = {};   // the symbol has one address per device
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return nullptr;
    if (ptrs[device] == nullptr) {
        void* addr = nullptr;
        if (cudaGetSymbolAddress(&addr, g_gemm_status) == cudaSuccess) ptrs[device] = static_cast<unsigned int*>(addr);
    }
    return ptrs[device];
}

int column_sum(void* out, const void* in, long long rows, long long cols, int accumulate, int dtype, cudaStream_t s) {
    CGPT_DISPATCH_DTYPE(dtype, T, {
        column_sum_kernel<T><<<static_cast<unsigned>((cols + 31) / 32), 256, 0, s>>>(
            static_cast<T*>(out), static_cast<const T*>(in), rows, static_cast<int>(cols), accumulate);
        count_launch();
        CGPT_LAUNCH_CHECK();
    });
    return CGPT_OK;
}

}  // namespace cgpt

using namespace cgpt;

extern "C" int cgpt_gemm(void* c, const void* a, const void* b, size_t m, size_t n, size_t k, int a_layout,
                         int b_layout, int accumulate, int dtype, int force_simt, cgpt_stream_t stream) {
    return gemm_dispatch(c, a, b, static_cast<long long>(m), static_cast<long long>(n), static_cast<long long>(k),
                         a_layout, b_layout, accumulate, dtype, force_simt != 0, static_cast<cudaStream_t>(stream));
}

extern "C" int cgpt_linear_forward(void* y, const void* x, const void* w, size_t rows, size_t in_features,
                                   size_t out_features, int dtype, cgpt_stream_t stream) {
    return gemm_dispatch(y, x, w, static_cast<long long>(rows), static_cast<long long>(out_features),
                         static_cast<long long>(in_features), 0, 0, 0, dtype, false, static_cast<cudaStream_t>(stream));
}

extern "C" int cgpt_linear_backward(void* dx, void* dw, void* db, const void* dy, const void* x, const void* w,
                                    size_t rows, size_t in_features, size_t out_features, int accumulate_input,
                                    int accumulate_weight, int accumulate_bias, int dtype, cgpt_stream_t stream) {
    if (!dy) return CGPT_ERR_NULL;
    auto s = static_cast<cudaStream_t>(stream);
    const long long T = static_cast<long long>(rows), I = static_cast<long long>(in_features), O = static_cast<long long>(out_features);
    if (dx != nullptr) {
        if (!w) return CGPT_ERR_NULL;
        CGPT_TRY(gemm_dispatch(dx, dy, w, T, I, O, 0, 1, accumulate_input, dtype, false, s));   // dX = dY * W
    }
    if (dw != nullptr) {
        if (!x) return CGPT_ERR_NULL;
        CGPT_TRY(gemm_dispatch(dw, dy, x, O, I, T, 1, 1, accumulate_weight, dtype, false, s));  // dW = dY^T * X
    }
    if (db != nullptr) {
        if (!valid_float_dtype(dtype) || T <= 0 || O <= 0) return CGPT_ERR_SHAPE;
        CGPT_TRY(column_sum(db, dy, T, O, accumulate_bias, dtype, s));
    }
    return CGPT_OK;
}

extern "C" int cgpt_linear_forward_fused(void* const* y, const void* x, const void* const* w, const size_t* out_features,
                                         size_t count, size_t rows, size_t in_features, int dtype, cgpt_stream_t stream) {
    if (!y || !x || !w || !out_features) return CGPT_ERR_NULL;
    if (count < 1 || count > static_cast<size_t>(kMaxKSegments)) return CGPT_ERR_SHAPE;
    auto s = static_cast<cudaStream_t>(stream);
    int ns[kMaxKSegments] = {0, 0, 0};
    for (size_t i = 0; i < count; ++i) {
        if (!y[i] || !w[i]) return CGPT_ERR_NULL;
        if (out_features[i] == 0 || out_features[i] > 0x7fffffffull) return CGPT_ERR_SHAPE;
        ns[i] = static_cast<int>(out_features[i]);
    }
    if (rows == 0 || in_features == 0 || rows > 0x7fffffffull || in_features > 0x7fffffffull) return CGPT_ERR_SHAPE;
    int rc = CGPT_ERR_UNSUPPORTED;
    if (pair_kernel_enabled()) {   // 256 x 256 tiles on CTA pairs where the shapes allow them
        if (dtype == CGPT_DTYPE_F16)
            rc = launch_tc_groups<__half, true>(reinterpret_cast<__half* const*>(y), static_cast<const __half*>(x),
                                                reinterpret_cast<const __half* const*>(w), ns, static_cast<int>(count), static_cast<int>(rows),
                                                static_cast<int>(in_features), dtype, s);
        else if (dtype == CGPT_DTYPE_BF16)
            rc = launch_tc_groups<__nv_bfloat16, true>(reinterpret_cast<__nv_bfloat16* const*>(y), static_cast<const __nv_bfloat16*>(x),
                                                       reinterpret_cast<const __nv_bfloat16* const*>(w), ns, static_cast<int>(count),
                                                       static_cast<int>(rows), static_cast<int>(in_features), dtype, s);
        if (rc != CGPT_ERR_UNSUPPORTED) return rc;
    }
    if (dtype == CGPT_DTYPE_F16)
        rc = launch_tc_groups<__half>(reinterpret_cast<__half* const*>(y), static_cast<const __half*>(x),
                                      reinterpret_cast<const __half* const*>(w), ns, static_cast<int>(count), static_cast<int>(rows),
                                      static_cast<int>(in_features), dtype, s);
    else if (dtype == CGPT_DTYPE_BF16)
        rc = launch_tc_groups<__nv_bfloat16>(reinterpret_cast<__nv_bfloat16* const*>(y), static_cast<const __nv_bfloat16*>(x),
                                             reinterpret_cast<const __nv_bfloat16* const*>(w), ns, static_cast<int>(count),
                                             static_cast<int>(rows), static_cast<int>(in_features), dtype, s);
    if (rc != CGPT_ERR_UNSUPPORTED) return rc;
    for (size_t i = 0; i < count; ++i)
        CGPT_TRY(gemm_dispatch(y[i], x, w[i], static_cast<long long>(rows), static_cast<long long>(out_features[i]),
                               static_cast<long long>(in_features), 0, 0, 0, dtype, false, s));
    return CGPT_OK;
}

extern "C" int cgpt_linear_backward_weight_fused(void* const* dw, const void* const* dy, const void* x, const size_t* out_features,
                                                 size_t count, size_t rows, size_t in_features, int accumulate_weight, int dtype,
                                                 cgpt_stream_t stream) {
    if (!dw || !dy || !x || !out_features) return CGPT_ERR_NULL;
    if (count < 1 || count > static_cast<size_t>(kMaxKSegments)) return CGPT_ERR_SHAPE;
    auto s = static_cast<cudaStream_t>(stream);
    int ms[kMaxKSegments] = {0, 0, 0};
    for (size_t i = 0; i < count; ++i) {
        if (!dw[i] || !dy[i]) return CGPT_ERR_NULL;
        if (out_features[i] == 0 || out_features[i] > 0x7fffffffull) return CGPT_ERR_SHAPE;
        ms[i] = static_cast<int>(out_features[i]);
    }
    if (rows == 0 || in_features == 0 || rows > 0x7fffffffull || in_features > 0x7fffffffull) return CGPT_ERR_SHAPE;
    int rc = CGPT_ERR_UNSUPPORTED;
    if (dtype == CGPT_DTYPE_F16)
        rc = launch_tc_mgroups<__half>(reinterpret_cast<__half* const*>(dw), reinterpret_cast<const __half* const*>(dy),
                                       static_cast<const __half*>(x), ms, static_cast<int>(count), static_cast<int>(in_features),
                                       static_cast<int>(rows), accumulate_weight, dtype, s);
    else if (dtype == CGPT_DTYPE_BF16)
        rc = launch_tc_mgroups<__nv_bfloat16>(reinterpret_cast<__nv_bfloat16* const*>(dw), reinterpret_cast<const __nv_bfloat16* const*>(dy),
                                              static_cast<const __nv_bfloat16*>(x), ms, static_cast<int>(count),
                                              static_cast<int>(in_features), static_cast<int>(rows), accumulate_weight, dtype, s);
    if (rc != CGPT_ERR_UNSUPPORTED) return rc;
    for (size_t i = 0; i < count; ++i)   // dW_i = dY_i^T X
        CGPT_TRY(gemm_dispatch(dw[i], dy[i], x, static_cast<long long>(out_features[i]), static_cast<long long>(in_features),
                               static_cast<long long>(rows), 1, 1, accumulate_weight, dtype, false, s));
    return CGPT_OK;
}

extern "C" int cgpt_linear_swiglu_forward(void* gate, void* up, void* activated, const void* x, const void* w_gate,
                                          const void* w_up, size_t rows, size_t in_features, size_t intermediate, int dtype,
                                          cgpt_stream_t stream) {
    return linear_swiglu_dispatch(gate, up, activated, x, w_gate, w_up, static_cast<long long>(rows),
                                  static_cast<long long>(intermediate), static_cast<long long>(in_features), dtype,
                                  static_cast<cudaStream_t>(stream));
}

extern "C" int cgpt_linear_backward_input_fused(void* dx, const void* const* dy, const void* const* w,
                                                const size_t* out_features, size_t count, size_t rows, size_t in_features,
                                                int accumulate_input, int dtype, cgpt_stream_t stream) {
    if (!dx || !dy || !w || !out_features) return CGPT_ERR_NULL;
    if (count < 1 || count > static_cast<size_t>(kMaxKSegments)) return CGPT_ERR_SHAPE;
    long long ks[kMaxKSegments] = {0, 0, 0};
    for (size_t i = 0; i < count; ++i) {
        if (!dy[i] || !w[i]) return CGPT_ERR_NULL;
        if (out_features[i] == 0 || out_features[i] > 0x7fffffffull) return CGPT_ERR_SHAPE;
        ks[i] = static_cast<long long>(out_features[i]);
    }
    if (rows == 0 || in_features == 0 || rows > 0x7fffffffull || in_features > 0x7fffffffull) return CGPT_ERR_SHAPE;
    // dX = sum_i dY_i * W_i: A_i = dY_i [rows, out_i] (K-major), B_i = W_i [out_i, in] read as [K, N]
    return gemm_dispatch_segments(dx, dy, w, ks, static_cast<int>(count), static_cast<long long>(rows),
                                  static_cast<long long>(in_features), 0, 1, accumulate_input, dtype, false,
                                  static_cast<cudaStream_t>(stream));
}

extern "C" int cgpt_linear_forward_sum(void* y, const void* const* x, const void* const* w, const size_t* in_features,
                                       size_t count, size_t rows, size_t out_features, const void* residual, int dtype,
                                       cgpt_stream_t stream) {
    if (!y || !x || !w || !in_features) return CGPT_ERR_NULL;
    if (count < 1 || count > static_cast<size_t>(kMaxKSegments)) return CGPT_ERR_SHAPE;
    long long ks[kMaxKSegments] = {0, 0, 0};
    for (size_t i = 0; i < count; ++i) {
        if (!x[i] || !w[i]) return CGPT_ERR_NULL;
        if (in_features[i] == 0 || in_features[i] > 0x7fffffffull) return CGPT_ERR_SHAPE;
        ks[i] = static_cast<long long>(in_features[i]);
    }
    if (rows == 0 || out_features == 0 || rows > 0x7fffffffull || out_features > 0x7fffffffull) return CGPT_ERR_SHAPE;
    auto s = static_cast<cudaStream_t>(stream);
    const long long T = static_cast<long long>(rows), O = static_cast<long long>(out_features);
    // Y = R + sum_i X_i W_i^T: A_i = X_i [rows, in_i], B_i = W_i [out, in_i], both K-major, chained along K
    int rc = gemm_dispatch_segments(y, x, w, ks, static_cast<int>(count), T, O, 0, 0, 0, dtype, false, s, residual);
    if (rc != CGPT_ERR_UNSUPPORTED || residual == nullptr) return rc;
    // no epilogue that adds the residual for this shape or dtype: the product alone, then one elementwise pass
    // (y may not alias the residual on this path: the product is written first)
    if (y == residual) return CGPT_ERR_OPTION;
    CGPT_TRY(gemm_dispatch_segments(y, x, w, ks, static_cast<int>(count), T, O, 0, 0, 0, dtype, false, s));
    return cgpt_add(y, y, residual, nullptr, rows * out_features, dtype, stream);
}

extern "C" int cgpt_b200_device_status(unsigned int* status_out, int clear) {
    if (!status_out) return CGPT_ERR_NULL;
    unsigned int v = 0;
    CGPT_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_gemm_status, sizeof(v)));
    if (clear && v != 0) {
        const unsigned int zero = 0;
        CGPT_CUDA_TRY(cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(zero)));
    }
    *status_out = v;
    return CGPT_OK;
}

extern "C" int cgpt_b200_gemm_timing(int enable) {
    g_timing.used = 0;
    g_timing.flops.clear();
    if (enable && g_timing.events.empty()) {
        g_timing.events.resize(8192);
        for (auto& e : g_timing.events) CGPT_CUDA_TRY(cudaEventCreate(&e));
    }
    g_timing.enabled = enable != 0;
    return CGPT_OK;
}

extern "C" int cgpt_b200_gemm_timing_read(double* total_ms, double* total_flops, uint64_t* launches) {
    if (!total_ms || !total_flops || !launches) return CGPT_ERR_NULL;
    CGPT_CUDA_TRY(cudaDeviceSynchronize());
    double ms = 0.0, fl = 0.0;
    for (std::size_t i = 0; i + 1 < g_timing.used; i += 2) {
        float t = 0.f;
        CGPT_CUDA_TRY(cudaEventElapsedTime(&t, g_timing.events[i], g_timing.events[i + 1]));
        ms += t;
        fl += g_timing.flops[i / 2];
    }
    *total_ms = ms;
    *total_flops = fl;
    *launches = g_timing.used / 2;
    return CGPT_OK;
}

// Tensor-core (tcgen05 / TMEM / TMA) attention kernels for sm_100a: 16-bit tensors, head_dim 64 or 128,
// any GQA ratio, causal (with query_position_offset) or full, Sq and Sk arbitrary.
//
// Forward (this file, first part): one CTA per (128-query tile, query head, batch).
//   warp 4      TMA producer: Q tile once, then K/V tiles of 128 keys through a 2-stage ring.
//   warp 5      MMA issuer: S = Q K^T (128x128xD) into one of two TMEM buffers, one tile ahead of the
//               softmax; PV = P V (128xDx128) into a third TMEM region once P is in shared memory.
//   warps 0-3   softmax: thread t owns query row t = TMEM lane t. Reads its S row from TMEM (two passes of
//               32-column chunks: row max, then exp2 and fp16 P written to 128B-swizzled shared memory as
//               the K-major A operand of the PV MMA), keeps the output row O (D fp32) and the running
//               max / sum in registers, and folds each PV tile in with the usual rescale.
// Numerics as the reference's tensor-core forward (src/ops/attention.cu:709-900): scores in the exp2
// domain (s * scale * log2 e), P rounded to the storage dtype before the PV product, fp32 O and sums,
// LSE = (max2 + log2(sum)) * ln 2 (natural log, scale included).
//
// All mbarrier waits are bounded (sm100::mbar_wait); a wait that runs out raises the library's device
// status word and the CTA leaves through the common exit (TMEM freed).
#include <type_traits>

#include "attention.h"
#include "launch_counter.h"
#include "sm100.cuh"

namespace cgpt {

// gemm.cu: device address of the status word shared by the tensor-core kernels (non-zero = a bounded wait ran out)
unsigned int* tc_status_device_ptr();

namespace {

using namespace sm100;

constexpr int kTile = 128;           // queries per CTA tile and keys per KV tile
constexpr int kFwdThreads = 192;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kMaskValue = -1.0e30f;

template <int D> struct FwdSmem {
    static constexpr int kChunks = D / 64;                 // 64-element (128-byte) column chunks of a [128, D] tile
    static constexpr int kTileBytes = kChunks * kTile * 128;
    static constexpr int kQ = 0;
    static constexpr int kK = kQ + kTileBytes;             // 2 stages
    static constexpr int kV = kK + 2 * kTileBytes;         // 2 stages
    static constexpr int kP = kV + 2 * kTileBytes;         // [128, 128] 16-bit = 2 chunks
    static constexpr int kBars = kP + 2 * kTile * 128;
    static constexpr int kBytes = kBars + 256 + 1024;      // + barriers + alignment slack
};

// Byte offset of 16-byte chunk `c16` (0..7) of row `row` inside a 128B-swizzled [rows][128 B] tile.
__device__ __forceinline__ std::uint32_t swz(int row, int c16) {
    return static_cast<std::uint32_t>(row * 128 + ((c16 ^ (row & 7)) << 4));
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

template <typename T, int D>
__global__ void __launch_bounds__(kFwdThreads, 1)
attention_forward_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                            const __grid_constant__ CUtensorMap tmap_v, T* __restrict__ out, float* __restrict__ lse,
                            AttnDims dm, unsigned int* __restrict__ status) {
    using L = FwdSmem<D>;
    extern __shared__ unsigned char attn_smem_raw[];
    const std::uint32_t raw = smem_u32(attn_smem_raw);
    unsigned char* smem = attn_smem_raw + ((1024u - (raw & 1023u)) & 1023u);
    std::uint64_t* bars = reinterpret_cast<std::uint64_t*>(smem + L::kBars);
    std::uint64_t* q_full = bars + 0;
    std::uint64_t* k_full = bars + 1;    // [2]
    std::uint64_t* v_full = bars + 3;    // [2]
    std::uint64_t* kv_empty = bars + 5;  // [2]
    std::uint64_t* s_full = bars + 7;    // [2]
    std::uint64_t* p_full = bars + 9;
    std::uint64_t* pv_full = bars + 10;
    std::uint32_t* tmem_slot = reinterpret_cast<std::uint32_t*>(bars + 11);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q_tiles = (dm.sq + kTile - 1) / kTile;
    const int q_tile = q_tiles - 1 - static_cast<int>(blockIdx.x);   // longest rows first
    const int h = blockIdx.y, b = blockIdx.z;
    const int kvh = h / (dm.hq / dm.hkv);
    const int q0 = q_tile * kTile;
    int q_last = q0 + kTile - 1;
    if (q_last > dm.sq - 1) q_last = dm.sq - 1;
    int last_key = dm.causal ? dm.offset + q_last : dm.sk - 1;
    if (last_key > dm.sk - 1) last_key = dm.sk - 1;
    const int n_kv = last_key / kTile + 1;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; ++s) { mbar_init(&k_full[s], 1); mbar_init(&v_full[s], 1); mbar_init(&kv_empty[s], 1); mbar_init(&s_full[s], 1); }
        mbar_init(p_full, kTile);
        mbar_init(pv_full, 1);
        mbar_init_fence();
        tma_prefetch_desc(&tmap_q); tma_prefetch_desc(&tmap_k); tma_prefetch_desc(&tmap_v);
    }
    if (warp == 5) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const std::uint32_t tmem = *tmem_slot;
    const std::uint32_t tmem_s[2] = {tmem, tmem + 128};
    const std::uint32_t tmem_pv = tmem + 256;
    bool failed = false;

    if (warp == 4) {
        if (lane == 0) {
            mbar_expect_tx(q_full, L::kTileBytes);
#pragma unroll
            for (int c = 0; c < L::kChunks; ++c) tma_load_4d(smem + L::kQ + c * kTile * 128, &tmap_q, q_full, c * 64, h, q0, b);
            for (int i = 0; i < n_kv; ++i) {
                const int s = i & 1;
                if (!mbar_wait(&kv_empty[s], ((i >> 1) & 1) ^ 1u)) { failed = true; break; }
                mbar_expect_tx(&k_full[s], L::kTileBytes);
#pragma unroll
                for (int c = 0; c < L::kChunks; ++c)
                    tma_load_4d(smem + L::kK + s * L::kTileBytes + c * kTile * 128, &tmap_k, &k_full[s], c * 64, kvh, i * kTile, b);
                mbar_expect_tx(&v_full[s], L::kTileBytes);
#pragma unroll
                for (int c = 0; c < L::kChunks; ++c)
                    tma_load_4d(smem + L::kV + s * L::kTileBytes + c * kTile * 128, &tmap_v, &v_full[s], c * 64, kvh, i * kTile, b);
            }
        }
    } else if (warp == 5) {
        if (lane == 0) {
            constexpr int fmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
            constexpr std::uint32_t idesc_s = idesc_f16(fmt, 0, 0, kTile, kTile);   // S: A = Q (K-major), B = K (K-major)
            constexpr std::uint32_t idesc_pv = idesc_f16(fmt, 0, 1, kTile, D);      // PV: A = P (K-major), B = V (N-major)
            const std::uint32_t q_base = smem_u32(smem + L::kQ);
            const std::uint32_t p_base = smem_u32(smem + L::kP);
            auto issue_s = [&](int i) {
                const std::uint32_t k_base = smem_u32(smem + L::kK + (i & 1) * L::kTileBytes);
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                    const std::uint32_t off = (k >> 2) * (kTile * 128) + (k & 3) * 32;
                    mma_f16_ss(tmem_s[i & 1], smem_desc_sw128(q_base + off, 16, 1024), smem_desc_sw128(k_base + off, 16, 1024),
                               idesc_s, k > 0 ? 1u : 0u);
                }
                tc_commit(&s_full[i & 1]);
            };
            if (!mbar_wait(q_full, 0) || !mbar_wait(&k_full[0], 0)) failed = true;
            if (!failed) {
                tc_fence_after_sync();
                issue_s(0);
                for (int i = 0; i < n_kv; ++i) {
                    if (i + 1 < n_kv) {
                        if (!mbar_wait(&k_full[(i + 1) & 1], ((i + 1) >> 1) & 1)) { failed = true; break; }
                        tc_fence_after_sync();
                        issue_s(i + 1);
                    }
                    if (!mbar_wait(&v_full[i & 1], (i >> 1) & 1) || !mbar_wait(p_full, i & 1)) { failed = true; break; }
                    tc_fence_after_sync();
                    const std::uint32_t v_base = smem_u32(smem + L::kV + (i & 1) * L::kTileBytes);
#pragma unroll
                    for (int k = 0; k < kTile / 16; ++k) {
                        const std::uint32_t a_off = (k >> 2) * (kTile * 128) + (k & 3) * 32;
                        mma_f16_ss(tmem_pv, smem_desc_sw128(p_base + a_off, 16, 1024),
                                   smem_desc_sw128(v_base + k * (16 * 128), kTile * 128, 1024), idesc_pv, k > 0 ? 1u : 0u);
                    }
                    tc_commit(pv_full);
                    tc_commit(&kv_empty[i & 1]);
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- softmax warps: thread = query row
        const int row = threadIdx.x;            // 0..127 = TMEM lane
        const int q_idx = q0 + row;
        const std::uint32_t lane_base = static_cast<std::uint32_t>(warp * 32) << 16;
        const float scale2 = dm.scale * kLog2e;
        float o_reg[D];
#pragma unroll
        for (int d = 0; d < D; ++d) o_reg[d] = 0.f;
        float m_run = kMaskValue, l_run = 0.f;
        unsigned char* p_smem = smem + L::kP;
        for (int i = 0; i < n_kv; ++i) {
            if (!mbar_wait(&s_full[i & 1], (i >> 1) & 1)) failed = true;
            failed = __any_sync(0xffffffffu, failed);
            if (failed) break;
            tc_fence_after_sync();
            const int kv0 = i * kTile;
            const bool need_mask = (kv0 + kTile > dm.sk) || (dm.causal && kv0 + kTile - 1 > dm.offset + q0);
            const int limit = dm.causal ? (dm.offset + q_idx < dm.sk - 1 ? dm.offset + q_idx : dm.sk - 1) : dm.sk - 1;  // last visible key
            // pass 1: row maximum
            float m_new = m_run;
#pragma unroll 1
            for (int c0 = 0; c0 < kTile; c0 += 32) {
                std::uint32_t r[32];
                tmem_ld_32x32(tmem_s[i & 1] + lane_base + c0, r);
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    float s2 = __uint_as_float(r[j]) * scale2;
                    if (need_mask && kv0 + c0 + j > limit) s2 = kMaskValue;
                    m_new = fmaxf(m_new, s2);
                }
            }
            const float alpha = exp2f(m_run - m_new);
            // pass 2: probabilities -> shared memory (K-major A operand of the PV product), row sum
            float row_sum = 0.f;
#pragma unroll 1
            for (int c0 = 0; c0 < kTile; c0 += 32) {
                std::uint32_t r[32];
                tmem_ld_32x32(tmem_s[i & 1] + lane_base + c0, r);
                std::uint32_t packed[16];
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    float a = __uint_as_float(r[j]) * scale2, bb = __uint_as_float(r[j + 1]) * scale2;
                    if (need_mask) {
                        if (kv0 + c0 + j > limit) a = kMaskValue;
                        if (kv0 + c0 + j + 1 > limit) bb = kMaskValue;
                    }
                    const float pa = exp2f(a - m_new), pb = exp2f(bb - m_new);
                    row_sum += pa + pb;
                    packed[j >> 1] = pack2<T>(pa, pb);
                }
                unsigned char* atom = p_smem + (c0 >> 6) * (kTile * 128);
                const int c16 = (c0 & 63) >> 3;
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4)
                    *reinterpret_cast<uint4*>(atom + swz(row, c16 + q4)) =
                        make_uint4(packed[4 * q4], packed[4 * q4 + 1], packed[4 * q4 + 2], packed[4 * q4 + 3]);
            }
            tc_fence_before_sync();      // TMEM reads of S done before the MMA warp may overwrite this buffer
            fence_proxy_async_smem();    // P visible to the tensor core's (async proxy) reads
            mbar_arrive(p_full);
            l_run = l_run * alpha + row_sum;
            m_run = m_new;
            if (!mbar_wait(pv_full, i & 1)) failed = true;
            failed = __any_sync(0xffffffffu, failed);
            if (failed) break;
            tc_fence_after_sync();
#pragma unroll
            for (int c0 = 0; c0 < D; c0 += 32) {
                std::uint32_t r[32];
                tmem_ld_32x32(tmem_pv + lane_base + c0, r);
#pragma unroll
                for (int j = 0; j < 32; ++j) o_reg[c0 + j] = fmaf(o_reg[c0 + j], alpha, __uint_as_float(r[j]));
            }
            tc_fence_before_sync();
        }
        if (!failed && q_idx < dm.sq) {
            const float inv = 1.0f / l_run;
            T* dst = out + ((static_cast<long long>(b) * dm.sq + q_idx) * dm.hq + h) * D;
#pragma unroll
            for (int d = 0; d < D; d += 8) {
                float v8[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) v8[e] = o_reg[d + e] * inv;
                store_vec<T, 8>(dst + d, v8);
            }
            if (lse != nullptr) lse[(static_cast<long long>(b) * dm.sq + q_idx) * dm.hq + h] = (m_run + log2f(l_run)) * kLn2;
        }
    }

    if (failed) {
        atomicExch(status, 1u);
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) { }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, 512);
    }
}

// 4D tensor map over a [batch, seq, heads, D] tensor: box = 64 columns x 1 head x 128 positions.
int make_bshd_map(CUtensorMap* map, const void* base, int dtype, int batch, int seq, int heads, int d) {
    const std::uint64_t dims[4] = {static_cast<std::uint64_t>(d), static_cast<std::uint64_t>(heads), static_cast<std::uint64_t>(seq),
                                   static_cast<std::uint64_t>(batch)};
    const std::uint64_t strides[3] = {static_cast<std::uint64_t>(d) * 2, static_cast<std::uint64_t>(heads) * d * 2,
                                      static_cast<std::uint64_t>(seq) * heads * d * 2};
    const std::uint32_t box[4] = {64, 1, kTile, 1};
    return make_tensor_map(map, dtype, base, 4, dims, strides, box);
}

template <typename T, int D>
int launch_forward(void* out, float* lse, const void* q, const void* k, const void* v, const AttnDims& dm, int dtype, cudaStream_t s) {
    using L = FwdSmem<D>;
    CUtensorMap tq, tk, tv;
    CGPT_TRY(make_bshd_map(&tq, q, dtype, dm.batch, dm.sq, dm.hq, D));
    CGPT_TRY(make_bshd_map(&tk, k, dtype, dm.batch, dm.sk, dm.hkv, D));
    CGPT_TRY(make_bshd_map(&tv, v, dtype, dm.batch, dm.sk, dm.hkv, D));
    auto kernel = attention_forward_tc_kernel<T, D>;
    static bool attr_done = false;
    if (!attr_done) {
        CGPT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes));
        attr_done = true;
    }
    unsigned int* status = tc_status_device_ptr();
    if (status == nullptr) return CGPT_ERR_STATE;
    const dim3 grid((dm.sq + kTile - 1) / kTile, dm.hq, dm.batch);
    kernel<<<grid, kFwdThreads, L::kBytes, s>>>(tq, tk, tv, static_cast<T*>(out), lse, dm, status);
    count_launch();
    CGPT_LAUNCH_CHECK();
    return CGPT_OK;
}

}  // namespace

int attention_forward_tc_launch(void* out, float* lse, const void* q, const void* k, const void* v, const AttnDims& dm,
                                int dtype, cudaStream_t s) {
    if (dtype == CGPT_DTYPE_F32 || (dm.d != 64 && dm.d != 128)) return CGPT_ERR_UNSUPPORTED;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out)) return CGPT_ERR_UNSUPPORTED;
    if (dm.hq > 65535 || dm.batch > 65535) return CGPT_ERR_UNSUPPORTED;
    if (dtype == CGPT_DTYPE_F16)
        return dm.d == 64 ? launch_forward<__half, 64>(out, lse, q, k, v, dm, dtype, s) : launch_forward<__half, 128>(out, lse, q, k, v, dm, dtype, s);
    return dm.d == 64 ? launch_forward<__nv_bfloat16, 64>(out, lse, q, k, v, dm, dtype, s)
                      : launch_forward<__nv_bfloat16, 128>(out, lse, q, k, v, dm, dtype, s);
}

}  // namespace cgpt

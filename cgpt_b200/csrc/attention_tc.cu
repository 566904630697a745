// Tensor-core (tcgen05 / TMEM / TMA) attention kernels for sm_100a: 16-bit tensors, head_dim 64 or 128,
// any GQA ratio, causal (with query_position_offset) or full, Sq and Sk arbitrary.
//
// Forward (this file, first part): one CTA per (128-query tile, query head, batch).
//   warp 8      TMA producer: Q tile once, then K/V tiles of 128 keys through a 2-stage ring.
//   warp 9      MMA issuer: S = Q K^T (128x128xD) into one of two TMEM buffers, one tile ahead of the
//               softmax; PV = P V (128xDx128) into a third TMEM region once P is in shared memory.
//   warps 0-7   softmax, two warpgroups: threads t and t+128 share query row t = TMEM lane t; each takes 64 of the
//               tile's 128 score columns (row max, exchanged with the partner through shared memory; then exp2 and
//               16-bit P written to 128B-swizzled shared memory as the K-major A operand of the PV MMA) and half of
//               the output row O (D/2 fp32 registers), folding each PV tile in with the usual rescale. The softmax
//               is a latency chain per tile, not an issue-rate problem: halving the chain per thread is what pays.
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
constexpr int kFwdThreads = 320;     // warps 0-7 softmax (two warpgroups, half of the tile's columns each), 8 TMA, 9 MMA
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
    static constexpr int kXchg = kP + 2 * kTile * 128;     // [2 parities + final][2 halves][128 rows] fp32, then a fail flag
    static constexpr int kBars = kXchg + 3 * 2 * kTile * 4 + 16;
    static constexpr int kBytes = kBars + 256 + 1024;      // + barriers + alignment slack
};

// Byte offset of 16-byte chunk `c16` (0..7) of row `row` inside a 128B-swizzled [rows][128 B] tile.
__device__ __forceinline__ std::uint32_t swz(int row, int c16) {
    return static_cast<std::uint32_t>(row * 128 + ((c16 ^ (row & 7)) << 4));
}

// 2^x on the special-function unit (flushes denormal results to zero, which is what a vanishing probability should be).
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

// 2^x for x <= 0 on the FMA and integer pipes: x = n + f with n = round(x) (read from the low mantissa bits of
// x + 1.5 * 2^23) and f in [-0.5, 0.5]; 2^f by a degree-3 polynomial (maximum relative error 7.5e-5, below the 4.9e-4 of the
// fp16 rounding P gets anyway); n is added to the exponent field. Pass 2 of the softmax is bound by the MUFU pipe
// (16 results per clock per SM against 128 FMAs), so a share of the exponentials is moved off it.
constexpr int kPolyEvery = 4;   // one pair in kPolyEvery uses the polynomial
__device__ __forceinline__ float poly_exp2(float x) {
    x = fmaxf(x, -125.0f);
    const float t = x + 12582912.0f;
    const float f = x - (t - 12582912.0f);
    float p = fmaf(f, 0.055171459913253784f, 0.2426108568906784f);
    p = fmaf(p, f, 0.6932609677314758f);
    p = fmaf(p, f, 0.9999281167984009f);
    return __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
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
    std::uint64_t* k_empty = bars + 5;   // [2] a K stage is free once the S product of its tile has completed ...
    std::uint64_t* v_empty = bars + 7;   // [2] ... a V stage only after the PV product, about one tile period later
    std::uint64_t* s_full = bars + 9;    // [2]
    std::uint64_t* p_full = bars + 11;
    std::uint64_t* pv_full = bars + 12;
    std::uint32_t* tmem_slot = reinterpret_cast<std::uint32_t*>(bars + 13);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q_tiles = (dm.sq + kTile - 1) / kTile;
    // 1-D grid, longest query tiles first over ALL (head, batch) pairs: the short tiles of the causal triangle fill the
    // tail of the launch.
    const int pairs = dm.hq * dm.batch;
    const int q_tile = q_tiles - 1 - static_cast<int>(blockIdx.x) / pairs;
    const int h = (static_cast<int>(blockIdx.x) % pairs) % dm.hq, b = (static_cast<int>(blockIdx.x) % pairs) / dm.hq;
    const int kvh = h / (dm.hq / dm.hkv);
    const int q0 = q_tile * kTile;
    int q_last = q0 + kTile - 1;
    if (q_last > dm.sq - 1) q_last = dm.sq - 1;
    int last_key = dm.causal ? dm.offset + q_last : dm.sk - 1;
    if (last_key > dm.sk - 1) last_key = dm.sk - 1;
    const int n_kv = last_key / kTile + 1;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; ++s) { mbar_init(&k_full[s], 1); mbar_init(&v_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_empty[s], 1); mbar_init(&s_full[s], 1); }
        mbar_init(p_full, 2 * kTile);
        mbar_init(pv_full, 1);
        mbar_init_fence();
        tma_prefetch_desc(&tmap_q); tma_prefetch_desc(&tmap_k); tma_prefetch_desc(&tmap_v);
    }
    if (warp == 9) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
    float* xchg = reinterpret_cast<float*>(smem + L::kXchg);
    volatile int* fail_flag = reinterpret_cast<volatile int*>(smem + L::kXchg + 3 * 2 * kTile * 4);
    if (threadIdx.x == 0) *fail_flag = 0;
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const std::uint32_t tmem = *tmem_slot;
    const std::uint32_t tmem_pv = tmem + 256;   // S buffers: columns [0,128) and [128,256), chosen by tile parity
    bool failed = false;

    if (warp == 8) {
        if (lane == 0) {
            mbar_expect_tx(q_full, L::kTileBytes);
#pragma unroll
            for (int c = 0; c < L::kChunks; ++c) tma_load_4d(smem + L::kQ + c * kTile * 128, &tmap_q, q_full, c * 64, h, q0, b);
            // Loads go out in the order their stages come free: K(i+1) (after S(i-1)) before V(i) (after PV(i-2)), so
            // the K tile the next S product needs is in flight a whole tile period before the MMA thread asks for it.
            auto load_k = [&](int i) -> bool {
                const int s = i & 1;
                if (!mbar_wait(&k_empty[s], ((i >> 1) & 1) ^ 1u)) return false;
                mbar_expect_tx(&k_full[s], L::kTileBytes);
#pragma unroll
                for (int c = 0; c < L::kChunks; ++c)
                    tma_load_4d(smem + L::kK + s * L::kTileBytes + c * kTile * 128, &tmap_k, &k_full[s], c * 64, kvh, i * kTile, b);
                return true;
            };
            if (!load_k(0)) failed = true;
            for (int i = 0; i < n_kv && !failed; ++i) {
                const int s = i & 1;
                if (i + 1 < n_kv && !load_k(i + 1)) { failed = true; break; }
                if (!mbar_wait(&v_empty[s], ((i >> 1) & 1) ^ 1u)) { failed = true; break; }
                mbar_expect_tx(&v_full[s], L::kTileBytes);
#pragma unroll
                for (int c = 0; c < L::kChunks; ++c)
                    tma_load_4d(smem + L::kV + s * L::kTileBytes + c * kTile * 128, &tmap_v, &v_full[s], c * 64, kvh, i * kTile, b);
            }
        }
    } else if (warp == 9) {
        if (lane == 0) {
            constexpr int fmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
            constexpr std::uint32_t idesc_s = idesc_f16(fmt, 0, 0, kTile, kTile);   // S: A = Q (K-major), B = K (K-major)
            constexpr std::uint32_t idesc_pv = idesc_f16(fmt, 0, 1, kTile, D);      // PV: A = P (K-major), B = V (N-major)
            // One thread issues every MMA, so the descriptors are built once; a K step or a ring stage only adds a
            // constant to the descriptor's 14-bit address field.
            constexpr std::uint32_t kStage16 = L::kTileBytes >> 4;
            const std::uint64_t q_desc = smem_desc_sw128(smem_u32(smem + L::kQ), 16, 1024);
            const std::uint64_t k_desc0 = smem_desc_sw128(smem_u32(smem + L::kK), 16, 1024);
            const std::uint64_t v_desc0 = smem_desc_sw128(smem_u32(smem + L::kV), kTile * 128, 1024);
            auto issue_s = [&](int i) {
                const std::uint64_t k_desc = k_desc0 + (i & 1) * kStage16;
                const std::uint32_t tmem_s = tmem + (i & 1) * 128;
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                    const std::uint32_t off16 = ((k >> 2) * (kTile * 128) + (k & 3) * 32) >> 4;
                    mma_f16_ss(tmem_s, q_desc + off16, k_desc + off16, idesc_s, k > 0 ? 1u : 0u);
                }
                tc_commit(&s_full[i & 1]);
                tc_commit(&k_empty[i & 1]);
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
                    const std::uint64_t v_desc = v_desc0 + (i & 1) * kStage16;
                    const std::uint32_t tmem_p = tmem + (i & 1) * 128;   // P over the tile's own score buffer
#pragma unroll
                    for (int k = 0; k < kTile / 16; ++k) {
                        // keys 16k..16k+15 = 8 packed columns; the two softmax warpgroups wrote keys 0-63 at columns
                        // [0,32) and keys 64-127 at columns [64,96)
                        const std::uint32_t a_col = (k >> 2) * 64 + (k & 3) * 8;
                        mma_f16_ts(tmem_pv, tmem_p + a_col, v_desc + ((k * (16 * 128)) >> 4), idesc_pv, k > 0 ? 1u : 0u);
                    }
                    tc_commit(pv_full);
                    tc_commit(&v_empty[i & 1]);
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- softmax warps
        // Two threads share a query row (= TMEM lane): warpgroup `half` handles columns [64*half, 64*half+64) of every
        // score tile and columns [D/2*half, ...) of the output row. Per tile they exchange their partial row maxima
        // through shared memory (one named barrier); the row sums stay partial until the end.
        const int row = threadIdx.x & (kTile - 1);
        const int half = threadIdx.x >> 7;
        const int q_idx = q0 + row;
        const std::uint32_t lane_base = static_cast<std::uint32_t>((warp & 3) * 32) << 16;
        const float scale2 = dm.scale * kLog2e;
        constexpr int DH = D / 2;
        float o_reg[DH];
#pragma unroll
        for (int d = 0; d < DH; ++d) o_reg[d] = 0.f;
        float m_run = kMaskValue, l_run = 0.f;
        // The PV product of tile i is folded into the output registers one step late, after pass 1 of tile i + 1: the
        // product then runs on the tensor core while these warps take the next tile's row maxima, instead of being
        // waited for. O = O * alpha_i + PV_i with alpha_i the rescale factor computed for tile i.
        float alpha_prev = 1.f;
        auto fold_pv = [&](int i) {
            if (!mbar_wait(pv_full, i & 1)) { failed = true; return; }
            tc_fence_after_sync();
#pragma unroll
            for (int c0 = 0; c0 < DH; c0 += 32) {
                std::uint32_t r[32];
                tmem_ld_32x32(tmem_pv + lane_base + half * DH + c0, r);
#pragma unroll
                for (int j = 0; j < 32; ++j) o_reg[c0 + j] = fmaf(o_reg[c0 + j], alpha_prev, __uint_as_float(r[j]));
            }
            tc_fence_before_sync();
        };
        for (int i = 0; i < n_kv; ++i) {
            if (!failed && !mbar_wait(&s_full[i & 1], (i >> 1) & 1)) failed = true;
            const int kv0 = i * kTile + half * 64;                    // first key of this thread's columns
            const bool need_mask = (kv0 + 64 > dm.sk) || (dm.causal && kv0 + 63 > dm.offset + q0);
            const int limit = dm.causal ? (dm.offset + q_idx < dm.sk - 1 ? dm.offset + q_idx : dm.sk - 1) : dm.sk - 1;  // last visible key
            const std::uint32_t tmem_s = tmem + (i & 1) * 128 + half * 64 + lane_base;
            float* my_slot = xchg + ((i & 1) * 2 + half) * kTile + row;
            const float* other_slot = xchg + ((i & 1) * 2 + (half ^ 1)) * kTile + row;
            // pass 1: maximum over this thread's 64 scores. Unmasked tiles take it on the raw scores (scale2 > 0).
            float m_part = kMaskValue;
            if (!failed) {
                tc_fence_after_sync();
                std::uint32_t r0[32], r1[32];
                tmem_ld_32x32_x2(tmem_s, r0, tmem_s + 32, r1);
                if (need_mask) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        m_part = fmaxf(m_part, kv0 + j > limit ? kMaskValue : __uint_as_float(r0[j]) * scale2);
                        m_part = fmaxf(m_part, kv0 + 32 + j > limit ? kMaskValue : __uint_as_float(r1[j]) * scale2);
                    }
                } else {
                    float raw_max = -3.0e38f;
#pragma unroll
                    for (int j = 0; j < 32; ++j) raw_max = fmaxf(raw_max, fmaxf(__uint_as_float(r0[j]), __uint_as_float(r1[j])));
                    m_part = raw_max * scale2;
                }
            } else {
                *fail_flag = 1;
            }
            *my_slot = m_part;
            asm volatile("bar.sync 1, 256;" ::: "memory");            // both halves published their maxima (or the flag)
            if (*fail_flag != 0) { failed = true; break; }             // uniform over the 256 threads
            const float m_new = fmaxf(m_run, fmaxf(m_part, *other_slot));
            const float alpha = fast_exp2(m_run - m_new);
            // tile i-1's product: folded now; its completion also says that the P buffer may be rewritten below. A wait
            // that gave up is reported at the next exchange (the stores below then go to a buffer nobody reads in time).
            if (i > 0) fold_pv(i - 1);
            // pass 2: p = 2^(s * scale2 - m) -> shared memory (K-major A operand of the PV product), partial row sum
            float row_sum = 0.f;
            const float neg_m = -m_new;
#pragma unroll 1
            for (int c0 = 0; c0 < 64; c0 += 32) {
                std::uint32_t r[32];
                tmem_ld_32x32(tmem_s + c0, r);
                std::uint32_t packed[16];
                // two straight-line variants (no branch inside the unrolled body: the exponentials of a chunk must be
                // free to overlap)
                if (need_mask) {
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        const float a = kv0 + c0 + j > limit ? kMaskValue : __uint_as_float(r[j]) * scale2;
                        const float bb = kv0 + c0 + j + 1 > limit ? kMaskValue : __uint_as_float(r[j + 1]) * scale2;
                        const float pa = fast_exp2(a + neg_m), pb = fast_exp2(bb + neg_m);
                        row_sum += pa + pb;
                        packed[j >> 1] = pack2<T>(pa, pb);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        // every kPolyEvery-th pair takes its exponentials from the FMA pipe instead of the MUFU pipe
                        const float xa = fmaf(__uint_as_float(r[j]), scale2, neg_m);
                        const float xb = fmaf(__uint_as_float(r[j + 1]), scale2, neg_m);
                        const bool poly = ((j >> 1) % kPolyEvery) == kPolyEvery - 1;
                        const float pa = poly ? poly_exp2(xa) : fast_exp2(xa);
                        const float pb = poly ? poly_exp2(xb) : fast_exp2(xb);
                        row_sum += pa + pb;
                        packed[j >> 1] = pack2<T>(pa, pb);
                    }
                }
                // P goes back into TMEM over this thread's own, already read, score columns: 16 packed words per chunk at
                // columns [c0/2, c0/2 + 16) of the thread's 64-column range. The PV product reads its A operand from there.
                tmem_st_32x16(tmem_s + (c0 >> 1), packed);
            }
            tmem_st_wait();
            tc_fence_before_sync();      // P written, S read: the MMA warp may use P and later overwrite this buffer
            mbar_arrive(p_full);
            l_run = l_run * alpha + row_sum;
            m_run = m_new;
            alpha_prev = alpha;
        }
        if (!failed && n_kv > 0) fold_pv(n_kv - 1);
        // total row sum = the two halves' partial sums (same order in both threads)
        if (failed) *fail_flag = 1;
        float* l_slots = xchg + 4 * kTile;   // own region: the per-tile slots may still be read by the partner
        l_slots[half * kTile + row] = l_run;
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (*fail_flag != 0) failed = true;
        if (!failed && q_idx < dm.sq) {
            const float l_total = l_slots[row] + l_slots[kTile + row];
            const float inv = 1.0f / l_total;
            T* dst = out + ((static_cast<long long>(b) * dm.sq + q_idx) * dm.hq + h) * D + half * DH;
#pragma unroll
            for (int d = 0; d < DH; d += 8) {
                float v8[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) v8[e] = o_reg[d + e] * inv;
                store_vec<T, 8>(dst + d, v8);
            }
            if (half == 0 && lse != nullptr) lse[(static_cast<long long>(b) * dm.sq + q_idx) * dm.hq + h] = (m_run + log2f(l_total)) * kLn2;
        }
    }

    if (failed) {
        atomicExch(status, 1u);
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) { }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 9) {
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
    static PerDeviceOnce attr_once;
    if (attr_once.needed()) {
        CGPT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes));
        attr_once.done();
    }
    unsigned int* status = tc_status_device_ptr();
    if (status == nullptr) return CGPT_ERR_STATE;
    const dim3 grid(static_cast<unsigned>(((dm.sq + kTile - 1) / kTile) * dm.hq * dm.batch));
    kernel<<<grid, kFwdThreads, L::kBytes, s>>>(tq, tk, tv, static_cast<T*>(out), lse, dm, status);
    count_launch();
    CGPT_LAUNCH_CHECK();
    return CGPT_OK;
}

}  // namespace

int attention_forward_tc_launch(void* out, float* lse, const void* q, const void* k, const void* v, const AttnDims& dm,
                                int dtype, cudaStream_t s) {
    if (dtype == CGPT_DTYPE_F32 || (dm.d != 64 && dm.d != 128)) return CGPT_ERR_UNSUPPORTED;
    if (!(dm.scale > 0.f)) return CGPT_ERR_UNSUPPORTED;   // the kernel takes row maxima before scaling
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out)) return CGPT_ERR_UNSUPPORTED;
    if (static_cast<long long>((dm.sq + kTile - 1) / kTile + (dm.sk + kTile - 1) / kTile) * dm.hq * dm.batch > 0x7fffffffll) return CGPT_ERR_UNSUPPORTED;   // 1-D grids
    if (dtype == CGPT_DTYPE_F16)
        return dm.d == 64 ? launch_forward<__half, 64>(out, lse, q, k, v, dm, dtype, s) : launch_forward<__half, 128>(out, lse, q, k, v, dm, dtype, s);
    return dm.d == 64 ? launch_forward<__nv_bfloat16, 64>(out, lse, q, k, v, dm, dtype, s)
                      : launch_forward<__nv_bfloat16, 128>(out, lse, q, k, v, dm, dtype, s);
}

}  // namespace cgpt

// CTA-pair variant of the persistent tcgen05 GEMM. Included by gemm.cu only (inside its anonymous namespace).
//
// Why: with one CTA per 128 x 256 tile every K step of 16 reads A (4 KB) and B (8 KB) from shared memory while TMA
// writes the same 12 KB for a later step: 24 KB per 128 tensor-core clocks = 192 B/clk against the 128 B/clk a
// shared memory delivers. The single-CTA kernel is therefore bound by shared-memory bandwidth at about two thirds of the
// tensor rate (measured: tensor pipe 72 % active). Here two CTAs of a cluster of 2 (the two SMs of a TPC) compute one
// 256 x 256 tile with tcgen05.mma.cta_group::2: each CTA holds its own 128 rows of A and HALF of B (128 of the 256
// columns), the hardware feeds both halves of B to both tensor cores, and each CTA accumulates its 128 x 256 half in its
// own TMEM. Per K step and CTA that is 8 KB read + 8 KB written = 128 B/clk: the same tile work with two thirds of
// the shared-memory traffic.
//
// Structure per CTA as in gemm_persistent.cuh: warp 0 = TMA producer (its own A rows and its own half of B; no load is
// multicast), warp 1 = TMEM allocation and, in the leader CTA (cluster rank 0) only, the MMA issue for the pair,
// warps 2-5 = epilogue of this CTA's 128 rows. Barriers:
//   full[s]       leader only. One arrival (the leader's producer, announcing the bytes of BOTH CTAs) + the transaction
//                 bytes of both CTAs' loads (the peer's loads name the leader's barrier through its cluster address).
//   empty[s]      one per CTA; the leader's MMA thread commits to both when the MMAs reading stage s have completed.
//   acc_full[b]   one per CTA; committed to both when a tile's accumulation has completed.
//   acc_empty[b]  leader only: 8 arrivals = the 4 epilogue warps of each CTA (the peer's arrive remotely).
// A cluster barrier brackets the kernel: nothing touches the other CTA's barriers or shared memory before both have
// initialised, and neither CTA exits (or frees TMEM) while the other may still signal it or read its operands.
// Every mbarrier wait is bounded as in the single-CTA kernel.
#pragma once

constexpr int kPairBM = 256;         // rows of a pair tile (128 per CTA)
constexpr int kPairBN = 256;
struct PairCfg {
    static constexpr int kStages = 6;
    static constexpr int kStoreBufs = 2;
    static constexpr int kABytes = BM * BK * 2;                  // this CTA's 128 rows
    static constexpr int kBBytes = (kPairBN / 2) * BK * 2;       // this CTA's half of the columns
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/ + kStoreBufs * BM * 128;
    static_assert(kSmemBytes <= 232448, "pair GEMM shared memory exceeds the 227 KB a CTA may use");
};

// Softmax work the epilogue can do on a 256 x 256 tile of LM-head logits while it is still in TMEM (the logits product of
// the cut cross-entropy). A thread of the epilogue owns one row of the tile, so row statistics need no exchange.
//   kSoftmaxStatsStore  store the 16-bit logits AND write, per row and tile, (max, sum exp(l - max)) over the tile's
//                       columns of the ROUNDED logits, plus the target's logit where the tile holds the target column
//   kSoftmaxStats       the same without storing the logits (pass 1 of the recomputing form)
//   kSoftmaxGrad        store G = (exp(l - row max) / row sum - onehot) * out_scale instead of the logits (pass 2)
// Per element the arithmetic is the row kernel's (cross_entropy_ring.cuh): logits rounded to the storage dtype,
// ex2.approx.ftz((l - max) * log2 e), non-target gradient e * (1/sum * out_scale), target (e * 1/sum - 1) * out_scale.
enum : int { kSoftmaxNone = 0, kSoftmaxStatsStore = 1, kSoftmaxStats = 2, kSoftmaxGrad = 3 };
struct SoftmaxEpilogue {
    float2* partial;                 // [M][tiles_n]
    float* target_logit;             // [M]; written for rows whose target column exists
    const std::uint32_t* targets;    // [M]
    const float2* row_stats;         // [M] (row max, 1 / row sum): kSoftmaxGrad only
    float out_scale;
};

template <typename T, bool A_MN, bool B_MN, int SOFTMAX>
__device__ __forceinline__ void gemm_pair_body(const GemmOperands& ops, const GemmOutputs& outs,
                         T* __restrict__ C, float* __restrict__ partial, int M, int N, int total_kb, int tiles_m,
                         int tiles_n, int splits, int kb_per_split, int epilogue, const SoftmaxEpilogue& sx) {
    using Cfg = PairCfg;
    constexpr int BN = kPairBN;
    extern __shared__ unsigned char gemm_smem_raw[];
    const std::uint32_t raw = smem_u32(gemm_smem_raw);
    unsigned char* smem = gemm_smem_raw + ((1024u - (raw & 1023u)) & 1023u);
    unsigned char* staging = smem + Cfg::kStages * Cfg::kStageBytes;
    std::uint64_t* bars = reinterpret_cast<std::uint64_t*>(staging + Cfg::kStoreBufs * BM * 128);
    std::uint64_t* full = bars;
    std::uint64_t* empty = bars + Cfg::kStages;
    std::uint64_t* acc_full = bars + 2 * Cfg::kStages;       // [2]
    std::uint64_t* acc_empty = bars + 2 * Cfg::kStages + 2;  // [2]
    std::uint32_t* tmem_slot = reinterpret_cast<std::uint32_t*>(bars + 2 * Cfg::kStages + 4);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const std::uint32_t rank = cluster_ctarank();          // 0 = leader
    const bool leader = rank == 0;
    const int pair = static_cast<int>(blockIdx.x >> 1);
    const int pairs = static_cast<int>(gridDim.x >> 1);
    const int tiles = tiles_m * tiles_n;
    const int units = tiles * splits;
    // Order of the work units. Column tiles fastest (default): the pairs running at the same time share a few row tiles of
    // A and the whole of a small B (a weight matrix). Row tiles fastest (kEpiRowTilesFastest, and every softmax epilogue):
    // for an LM-head-shaped product, where B (the vocabulary matrix) is the large operand, the running pairs share a few
    // column tiles of B and B streams from memory once instead of once per row tile (measured on the 8192 x 32000 x 1024
    // logits product: DRAM traffic 1.23 GB -> its algorithmic 0.6 GB, the loss layer 7 % faster).
    const bool m_fastest = SOFTMAX != kSoftmaxNone || (epilogue & kEpiRowTilesFastest) != 0;
    epilogue &= ~kEpiRowTilesFastest;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); }
        mbar_init_fence();
        for (int i = 0; i < ops.segments; ++i) { tma_prefetch_desc(&ops.a[i]); tma_prefetch_desc(&ops.b[i]); }
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, 2 * BN);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    cluster_sync_all();            // both CTAs: barriers initialised, TMEM allocated
    tc_fence_after_sync();
    const std::uint32_t tmem_base = *tmem_slot;
    bool failed = false;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            for (int u = pair; u < units && !failed; u += pairs) {
                const int split = u / tiles, t = u % tiles;
                const int tile_m = m_fastest ? t % tiles_m : t / tiles_n;
                const int tile_n = m_fastest ? t / tiles_m : t % tiles_n;
                const int kb_begin = split * kb_per_split;
                int nkb = total_kb - kb_begin;
                if (nkb > kb_per_split) nkb = kb_per_split;
                const int tile_g = ops.group_dim ? tile_m : tile_n;
                int group = 0, tile_first = 0;
                if (ops.groups > 1 && tile_g >= ops.tile_end[0]) { group = 1; tile_first = ops.tile_end[0]; }
                if (ops.groups > 2 && tile_g >= ops.tile_end[1]) { group = 2; tile_first = ops.tile_end[1]; }
                const int n0 = (ops.group_dim ? tile_n : tile_n - tile_first) * BN + static_cast<int>(rank) * (BN / 2);   // this CTA's columns of B
                const int m0 = (ops.group_dim ? tile_m - tile_first : tile_m) * kPairBM + static_cast<int>(rank) * BM;    // this CTA's rows of A
                for (int i = 0; i < nkb; ++i, ++it) {
                    const int s = it % Cfg::kStages;
                    const std::uint32_t ph = (it / Cfg::kStages) & 1;
                    if (!mbar_wait(&empty[s], ph ^ 1u)) { failed = true; break; }
                    // the leader announces the bytes of both CTAs; both CTAs' loads complete on the leader's barrier
                    if (leader) mbar_expect_tx(&full[s], 2 * Cfg::kStageBytes);
                    const std::uint32_t bar = mapa_shared(smem_u32(&full[s]), 0);
                    unsigned char* a_dst = smem + s * Cfg::kStageBytes;
                    unsigned char* b_dst = a_dst + Cfg::kABytes;
                    const int kb = kb_begin + i;
                    int seg = 0, kb_first = 0;
                    if (ops.segments > 1 && kb >= ops.kb_end[0]) { seg = 1; kb_first = ops.kb_end[0]; }
                    if (ops.segments > 2 && kb >= ops.kb_end[1]) { seg = 2; kb_first = ops.kb_end[1]; }
                    const CUtensorMap* tmap_a = &ops.a[ops.groups > 1 ? group : seg];
                    const CUtensorMap* tmap_b = &ops.b[ops.groups > 1 ? group : seg];
                    const int k0 = (kb - kb_first) * BK;
                    if (!A_MN) {
                        tma_load_2d_pair(a_dst, tmap_a, bar, k0, m0);
                    } else {
#pragma unroll
                        for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(a_dst + j * (BK * 128), tmap_a, bar, m0 + j * 64, k0);
                    }
                    if (!B_MN) {
                        tma_load_2d_pair(b_dst, tmap_b, bar, k0, n0);
                    } else {
#pragma unroll
                        for (int j = 0; j < (BN / 2) / 64; ++j) tma_load_2d_pair(b_dst + j * (BK * 128), tmap_b, bar, n0 + j * 64, k0);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            constexpr std::uint32_t idesc = idesc_f16(std::is_same<T, __nv_bfloat16>::value ? 1 : 0, A_MN ? 1 : 0, B_MN ? 1 : 0, kPairBM, BN);
            int it = 0, j = 0;
            for (int u = pair; u < units && !failed; u += pairs, ++j) {
                const int split = u / tiles;
                const int kb_begin = split * kb_per_split;
                int nkb = total_kb - kb_begin;
                if (nkb > kb_per_split) nkb = kb_per_split;
                const int buf = j & 1;
                if (!mbar_wait(&acc_empty[buf], ((j >> 1) & 1) ^ 1u)) { failed = true; break; }
                tc_fence_after_sync();
                const std::uint32_t tmem_acc = tmem_base + buf * BN;
                for (int i = 0; i < nkb; ++i, ++it) {
                    const int s = it % Cfg::kStages;
                    const std::uint32_t ph = (it / Cfg::kStages) & 1;
                    if (!mbar_wait(&full[s], ph)) { failed = true; break; }
                    tc_fence_after_sync();
                    const std::uint32_t a_base = smem_u32(smem + s * Cfg::kStageBytes);
                    const std::uint32_t b_base = a_base + Cfg::kABytes;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const std::uint64_t adesc = A_MN ? smem_desc_sw128(a_base + k * (UMMA_K * 128), BK * 128, 1024)
                                                         : smem_desc_sw128(a_base + k * (UMMA_K * 2), 16, 1024);
                        const std::uint64_t bdesc = B_MN ? smem_desc_sw128(b_base + k * (UMMA_K * 128), BK * 128, 1024)
                                                         : smem_desc_sw128(b_base + k * (UMMA_K * 2), 16, 1024);
                        mma_f16_ss_pair(tmem_acc, adesc, bdesc, idesc, (i > 0 || k > 0) ? 1u : 0u);
                    }
                    // stage s is free in both CTAs once these MMAs have completed
                    const std::uint32_t e_local = smem_u32(&empty[s]);
                    tc_commit_pair(e_local);
                    tc_commit_pair(mapa_shared(e_local, 1));
                }
                const std::uint32_t f_local = smem_u32(&acc_full[buf]);
                tc_commit_pair(f_local);
                tc_commit_pair(mapa_shared(f_local, 1));
            }
        }
    } else {
        const int quarter = warp & 3;
        int j = 0;
        int stage_buf = 0;
        for (int u = pair; u < units; u += pairs, ++j) {
            const int split = u / tiles, t = u % tiles;
            const int tile_m = m_fastest ? t % tiles_m : t / tiles_n;
            const int tile_n = m_fastest ? t / tiles_m : t % tiles_n;
            const int buf = j & 1;
            if (!mbar_wait(&acc_full[buf], (j >> 1) & 1)) failed = true;
            failed = __any_sync(0xffffffffu, failed);
            if (failed) break;
            tc_fence_after_sync();
            const int row = tile_m * kPairBM + static_cast<int>(rank) * BM + quarter * 32 + lane;
            const std::uint32_t tmem_acc = tmem_base + buf * BN + (static_cast<std::uint32_t>(quarter * 32) << 16);
            if constexpr (SOFTMAX != kSoftmaxNone) {
                constexpr bool kStores = SOFTMAX != kSoftmaxStats;
                const int et = threadIdx.x - 64;
                const int trow = quarter * 32 + lane;
                const bool row_ok = row < M;
                const std::uint32_t tgt = row_ok ? sx.targets[row] : 0xffffffffu;
                const long long rel = static_cast<long long>(tgt) - static_cast<long long>(tile_n) * BN;
                // the target's column inside this tile, or -1 (other tile, or no valid target)
                const int tgt_rel = (tgt < static_cast<std::uint32_t>(N) && rel >= 0 && rel < BN) ? static_cast<int>(rel) : -1;
                float run_m = -3.0e38f, run_s = 0.f, target_value = 0.f;
                float row_max = 0.f, inv_sum = 0.f;
                if (SOFTMAX == kSoftmaxGrad && row_ok) {
                    const float2 st = sx.row_stats[row];
                    row_max = st.x;
                    inv_sum = st.y;
                }
                const float k = inv_sum * sx.out_scale;
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 64) {
                    unsigned char* buf_s = staging + stage_buf * (BM * 128);
                    if (kStores) {
                        if (et == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                    }
                    std::uint32_t r0[32], r1[32];
                    tmem_ld_32x32_x2(tmem_acc + c0, r0, tmem_acc + c0 + 32, r1);
                    float v[64];
#pragma unroll
                    for (int e = 0; e < 32; ++e) { v[e] = __uint_as_float(r0[e]); v[32 + e] = __uint_as_float(r1[e]); }
                    // the values a materialised logits tensor would hold
#pragma unroll
                    for (int e = 0; e < 64; e += 2) round_pair_to_storage<T>(v[e], v[e + 1]);
                    const int ncols = N - (tile_n * BN + c0);     // columns of this chunk that exist
                    const bool hit = tgt_rel >= c0 && tgt_rel < c0 + 64;
                    if (hit) {
#pragma unroll
                        for (int e = 0; e < 64; ++e)
                            if (c0 + e == tgt_rel) target_value = v[e];
                    }
                    if (SOFTMAX != kSoftmaxGrad) {
                        if (ncols > 0) {
                            if (ncols < 64) {
#pragma unroll
                                for (int e = 0; e < 64; ++e)
                                    if (e >= ncols) v[e] = -3.0e38f;
                            }
                            float m4[4] = {v[0], v[1], v[2], v[3]};
#pragma unroll
                            for (int e = 4; e < 64; ++e) m4[e & 3] = fmaxf(m4[e & 3], v[e]);
                            const float new_m = fmaxf(fmaxf(run_m, fmaxf(m4[0], m4[1])), fmaxf(m4[2], m4[3]));
                            float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                            for (int e = 0; e < 64; ++e) s4[e & 3] += fast_exp(v[e] - new_m);
                            run_s = run_s * fast_exp(run_m - new_m) + ((s4[0] + s4[1]) + (s4[2] + s4[3]));
                            run_m = new_m;
                            if (ncols < 64) {   // the store below must not see the mask (TMA clips the columns anyway)
#pragma unroll
                                for (int e = 0; e < 64; ++e)
                                    if (e >= ncols) v[e] = 0.f;
                            }
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < 64; ++e) v[e] = fast_exp(v[e] - row_max) * k;
                        if (hit) {
                            const float g = (fast_exp(target_value - row_max) * inv_sum - 1.0f) * sx.out_scale;
#pragma unroll
                            for (int e = 0; e < 64; ++e)
                                if (c0 + e == tgt_rel) v[e] = g;
                        }
                    }
                    if (kStores) {
#pragma unroll
                        for (int jj = 0; jj < 8; ++jj) {
                            float w[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e) w[e] = v[8 * jj + e];
                            store_vec<T, 8>(reinterpret_cast<T*>(buf_s + trow * 128 + ((jj ^ (trow & 7)) << 4)), w);
                        }
                        fence_proxy_async_smem();
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                        if (et == 0) {
                            const int cx = tile_n * BN + c0;
                            const int cy = tile_m * kPairBM + static_cast<int>(rank) * BM;
                            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                                         ::"l"(reinterpret_cast<std::uint64_t>(&outs.c[0])), "r"(smem_u32(buf_s)), "r"(cx), "r"(cy)
                                         : "memory");
                            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                        }
                        stage_buf ^= 1;
                    }
                }
                if (SOFTMAX != kSoftmaxGrad && row_ok) {
                    sx.partial[static_cast<long long>(row) * tiles_n + tile_n] = make_float2(run_m, run_s);
                    if (tgt_rel >= 0) sx.target_logit[row] = target_value;
                }
            } else if (epilogue == kEpiStoreTma || epilogue == kEpiStoreTmaResidual) {
                const int et = threadIdx.x - 64;
                const int trow = quarter * 32 + lane;
                // kEpiStoreTmaResidual: C points at a [M, N] tensor that is added to the product in fp32 before the one
                // rounding (N % 64 == 0, checked by the host: a chunk of 64 columns is inside the row or outside it)
                const bool with_residual = epilogue == kEpiStoreTmaResidual;
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 64) {
                    unsigned char* buf_s = staging + stage_buf * (BM * 128);
                    uint4 res[8];
                    const bool res_ok = with_residual && row < M && tile_n * BN + c0 < N;
                    if (res_ok) {     // issued before the waits below: the loads fly under them
                        const uint4* rp = reinterpret_cast<const uint4*>(C + static_cast<long long>(row) * N + tile_n * BN + c0);
#pragma unroll
                        for (int jj = 0; jj < 8; ++jj) res[jj] = __ldg(rp + jj);
                    }
                    if (et == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    std::uint32_t r0[32], r1[32];
                    tmem_ld_32x32_x2(tmem_acc + c0, r0, tmem_acc + c0 + 32, r1);
#pragma unroll
                    for (int jj = 0; jj < 8; ++jj) {
                        const std::uint32_t* src = jj < 4 ? &r0[8 * jj] : &r1[8 * (jj - 4)];
                        float v[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(src[e]);
                        if (res_ok) {
                            Pack<T, 8> pk;
                            *reinterpret_cast<uint4*>(&pk) = res[jj];
                            float rv[8];
                            unpack_pack(rv, pk);
#pragma unroll
                            for (int e = 0; e < 8; ++e) v[e] += rv[e];
                        }
                        store_vec<T, 8>(reinterpret_cast<T*>(buf_s + trow * 128 + ((jj ^ (trow & 7)) << 4)), v);
                    }
                    fence_proxy_async_smem();
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (et == 0) {
                        const int tile_g = ops.group_dim ? tile_m : tile_n;
                        int group = 0, tile_first = 0;
                        if (ops.groups > 1 && tile_g >= ops.tile_end[0]) { group = 1; tile_first = ops.tile_end[0]; }
                        if (ops.groups > 2 && tile_g >= ops.tile_end[1]) { group = 2; tile_first = ops.tile_end[1]; }
                        const int cx = (ops.group_dim ? tile_n : tile_n - tile_first) * BN + c0;
                        const int cy = (ops.group_dim ? tile_m - tile_first : tile_m) * kPairBM + static_cast<int>(rank) * BM;
                        asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                                     ::"l"(reinterpret_cast<std::uint64_t>(&outs.c[group])), "r"(smem_u32(buf_s)), "r"(cx), "r"(cy)
                                     : "memory");
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                    stage_buf ^= 1;
                }
            } else {
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 64) {
                    std::uint32_t r0[32], r1[32];
                    tmem_ld_32x32_x2(tmem_acc + c0, r0, tmem_acc + c0 + 32, r1);
                    gemm_store_chunk<T>(r0, C, partial, row, tile_n * BN + c0, M, N, split, epilogue);
                    gemm_store_chunk<T>(r1, C, partial, row, tile_n * BN + c0 + 32, M, N, split, epilogue);
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&acc_empty[buf]), 0));   // the leader's barrier counts both CTAs
        }
    }

    if (threadIdx.x == 64) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    if (failed) {
        atomicExch(&g_gemm_status, 1u);
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) { }
    }
    tc_fence_before_sync();
    cluster_sync_all();            // neither CTA leaves while the other may still read its operands or signal its barriers
    if (warp == 1) {
        __syncwarp();              // the deallocation is a warp-wide (.sync.aligned) instruction
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, 2 * BN);
    }
}

template <typename T, bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ GemmOperands ops, const __grid_constant__ GemmOutputs outs,
                         T* __restrict__ C, float* __restrict__ partial, int M, int N, int total_kb, int tiles_m,
                         int tiles_n, int splits, int kb_per_split, int epilogue) {
    const SoftmaxEpilogue none{nullptr, nullptr, nullptr, nullptr, 0.f};
    gemm_pair_body<T, A_MN, B_MN, kSoftmaxNone>(ops, outs, C, partial, M, N, total_kb, tiles_m, tiles_n, splits, kb_per_split,
                                                epilogue, none);
}

// The LM-head product X C^T (both operands K-major, no split-K) with one of the softmax epilogues.
template <typename T, int SOFTMAX>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_pair_softmax_kernel(const __grid_constant__ GemmOperands ops, const __grid_constant__ GemmOutputs outs, int M, int N,
                         int total_kb, int tiles_m, int tiles_n, const SoftmaxEpilogue sx) {
    gemm_pair_body<T, false, false, SOFTMAX>(ops, outs, nullptr, nullptr, M, N, total_kb, tiles_m, tiles_n, 1, total_kb,
                                             kEpiStoreTma, sx);
}

// Grid of the pair kernel: two CTAs per cluster, one cluster per TPC that can host it.
inline int pair_grid(const void* kernel, int units) {
    static int max_pairs[64] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 0;
    if (max_pairs[device] == 0) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(kNumSMs, 1, 1);
        cfg.blockDim = dim3(kGemmThreads, 1, 1);
        cfg.dynamicSmemBytes = PairCfg::kSmemBytes;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess || clusters <= 0) {
            cudaGetLastError();
            max_pairs[device] = -1;
        } else {
            max_pairs[device] = clusters < kNumSMs / 2 ? clusters : kNumSMs / 2;
        }
    }
    if (max_pairs[device] <= 0) return 0;
    const int p = units < max_pairs[device] ? units : max_pairs[device];
    return 2 * p;
}

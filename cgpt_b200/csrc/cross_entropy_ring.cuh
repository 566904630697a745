// Cross-entropy over materialised 16-bit logits with an asynchronous row ring. Included by cross_entropy.cu only.
//
// One persistent CTA of 1024 threads per SM walks rows blockIdx.x, blockIdx.x + grid, ... Rows arrive in a ring of
// 2-3 shared-memory buffers through untiled bulk copies (cp.async.bulk + mbarrier), issued `stages` rows ahead by one
// thread, so HBM reads run underneath the arithmetic of earlier rows. A thread lifts its (up to) 4 chunks of 8 logits
// out of shared memory ONCE into fp32 registers; the row maximum, exp(logit - max) (computed once: the registers are
// overwritten with it), the row sum and the gradient all come from those registers, and the gradient goes straight
// from registers to global memory. Per element: one shared-memory read, one MUFU, one global write.
// Per element the arithmetic is the reference's fast-math build: ex2.approx.ftz((logit - max) * log2 e), probabilities
// times 1/sum; the non-target gradient folds 1/sum and the output scale into one factor (one fp32 rounding fewer).
#pragma once

constexpr int kRingThreads = 1024;         // one CTA per SM: 64 registers per thread
constexpr int kRingWarps = kRingThreads / 32;
constexpr int kRingCpt = 4;                // 16-byte chunks per thread held in registers (32 fp32 values)

// Packed pair arithmetic on the storage dtype.
template <typename T> struct Packed2;
template <> struct Packed2<__half> {
    using type = __half2;
    static __device__ __forceinline__ type from(std::uint32_t u) { return *reinterpret_cast<const __half2*>(&u); }
    static __device__ __forceinline__ type max(type a, type b) { return __hmax2(a, b); }
    static __device__ __forceinline__ type lowest() { return from(0xfbfffbffu); }          // -65504 twice
    static __device__ __forceinline__ uint4 lowest_raw4() { return make_uint4(0xfbfffbffu, 0xfbfffbffu, 0xfbfffbffu, 0xfbfffbffu); }
    static __device__ __forceinline__ float hmax(type a) { return fmaxf(__low2float(a), __high2float(a)); }
};
template <> struct Packed2<__nv_bfloat16> {
    using type = __nv_bfloat162;
    static __device__ __forceinline__ type from(std::uint32_t u) { return *reinterpret_cast<const __nv_bfloat162*>(&u); }
    static __device__ __forceinline__ type max(type a, type b) { return __hmax2(a, b); }
    static __device__ __forceinline__ type lowest() { return from(0xff7fff7fu); }          // lowest finite bf16 twice
    static __device__ __forceinline__ uint4 lowest_raw4() { return make_uint4(0xff7fff7fu, 0xff7fff7fu, 0xff7fff7fu, 0xff7fff7fu); }
    static __device__ __forceinline__ float hmax(type a) { return fmaxf(__low2float(a), __high2float(a)); }
};

// Block-wide reductions over kRingThreads threads, combined in a fixed order.
__device__ __forceinline__ float ring_block_max(float v, float* red) {
    v = warp_max(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = red[0];
#pragma unroll
    for (int i = 1; i < kRingWarps; ++i) r = fmaxf(r, red[i]);
    return r;
}
__device__ __forceinline__ float ring_block_sum(float v, float* red) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = 0.f;
#pragma unroll
    for (int i = 0; i < kRingWarps; ++i) r += red[i];
    return r;
}
constexpr int kRingMaxVocab = kRingThreads * kRingCpt * 8;
constexpr int kRingMaxStages = 3;
constexpr std::size_t kRingSmemBudget = 200 * 1024;

template <typename T>
__global__ void __launch_bounds__(kRingThreads, 1)
cross_entropy_ring_kernel(float* __restrict__ row_loss, T* grad, const T* logits, const std::uint32_t* __restrict__ targets,
                          long long rows, int vocab, float inv_rows, float gradient_scale, int stages, unsigned row_pitch,
                          unsigned int* __restrict__ status) {
    extern __shared__ __align__(128) unsigned char ce_ring[];
    __shared__ float red[kRingWarps];
    __shared__ std::uint64_t full[kRingMaxStages];
    const unsigned row_bytes = static_cast<unsigned>(vocab) * sizeof(T);
    const int chunks = vocab / 8;
    const long long first = blockIdx.x;
    const long long my_rows = first < rows ? (rows - first + gridDim.x - 1) / gridDim.x : 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) sm100::mbar_init(&full[s], 1);
        sm100::mbar_init_fence();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages && s < my_rows; ++s) {
            sm100::mbar_expect_tx(&full[s], row_bytes);
            sm100::bulk_load_1d(ce_ring + static_cast<std::size_t>(s) * row_pitch, logits + (first + s * static_cast<long long>(gridDim.x)) * vocab,
                                row_bytes, &full[s]);
        }
    }

    int stage = 0;
    std::uint32_t parity = 0;
    for (long long i = 0; i < my_rows; ++i) {
        const long long row = first + i * gridDim.x;
        const std::uint32_t target = targets[row];   // issued before the wait: its latency hides behind the two row passes
        const int failed = __syncthreads_or(sm100::mbar_wait(&full[stage], parity) ? 0 : 1);
        if (failed) {
            if (threadIdx.x == 0) atomicExch(status, 4u);
            const unsigned long long t0 = sm100::globaltimer_ns();
            while (sm100::globaltimer_ns() - t0 < 200000ull) { }   // let copies still in flight land before the CTA's memory goes away
            break;   // uniform: every thread saw the same value
        }
        const T* staged = reinterpret_cast<const T*>(ce_ring + static_cast<std::size_t>(stage) * row_pitch);

        // row maximum on the packed 16-bit values (exact in any format), two elements per instruction
        uint4 raw[kRingCpt];
        typename Packed2<T>::type m2 = Packed2<T>::lowest();
#pragma unroll
        for (int c = 0; c < kRingCpt; ++c) {
            const int chunk = c * kRingThreads + threadIdx.x;
            raw[c] = chunk < chunks ? *reinterpret_cast<const uint4*>(staged + chunk * 8) : Packed2<T>::lowest_raw4();
            m2 = Packed2<T>::max(m2, Packed2<T>::max(Packed2<T>::max(Packed2<T>::from(raw[c].x), Packed2<T>::from(raw[c].y)),
                                                     Packed2<T>::max(Packed2<T>::from(raw[c].z), Packed2<T>::from(raw[c].w))));
        }
        const float maximum = ring_block_max(Packed2<T>::hmax(m2), red);
        // e = exp(logit - max), computed once and kept; the padding (lowest finite value) gives exactly 0
        float v[kRingCpt][8];
        float local_sum = 0.f;
#pragma unroll
        for (int c = 0; c < kRingCpt; ++c) {
            Pack<T, 8> pk;
            *reinterpret_cast<uint4*>(&pk) = raw[c];
            unpack_pack(v[c], pk);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                v[c][e] = fast_exp(v[c][e] - maximum);
                local_sum += v[c][e];
            }
        }
        const float denominator = ring_block_sum(local_sum, red);
        const float inv_denominator = __frcp_rn(denominator);
        const bool valid = target < static_cast<std::uint32_t>(vocab);
        if (threadIdx.x == 0)
            row_loss[row] = valid ? (__logf(denominator) + maximum - to_f32<T>(staged[target])) * inv_rows : 0.f;
        if (grad != nullptr) {
            T* dst = grad + row * vocab;
            const float out_scale = inv_rows * gradient_scale;
            const float k = inv_denominator * out_scale;
#pragma unroll
            for (int c = 0; c < kRingCpt; ++c) {
                const int chunk = c * kRingThreads + threadIdx.x;
                if (chunk < chunks) {
                    float p[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) p[e] = v[c][e] * k;
                    store_vec<T, 8>(dst + chunk * 8, p);
                }
            }
            // The one element that carries the -1 is rewritten by the thread that owns its chunk (same thread, same
            // address, program order: this store lands after the vector store above).
            if (valid && static_cast<int>((target >> 3) % kRingThreads) == static_cast<int>(threadIdx.x)) {
                const float e = fast_exp(to_f32<T>(staged[target]) - maximum);
                dst[target] = from_f32<T>((e * inv_denominator - 1.0f) * out_scale);
            }
        }
        __syncthreads();   // every read of this ring buffer (thread 0's target lookup included) is done
        if (threadIdx.x == 0 && i + stages < my_rows) {
            sm100::mbar_expect_tx(&full[stage], row_bytes);
            sm100::bulk_load_1d(ce_ring + static_cast<std::size_t>(stage) * row_pitch, logits + (row + static_cast<long long>(stages) * gridDim.x) * vocab,
                                row_bytes, &full[stage]);
        }
        if (++stage == stages) { stage = 0; parity ^= 1u; }
    }
}

// Stages that fit, or 0 when the ring kernel does not apply to this shape.
template <typename T>
int ring_stages(long long vocab, const void* logits, const void* grad, unsigned* row_pitch) {
    static const bool enabled = [] {
        const char* e = diagnosis_env("CGPT_B200_CE_RING");   // diagnosis builds: "0" keeps the plain staged kernel
        return !(e != nullptr && e[0] == '0');
    }();
    if (!enabled || sizeof(T) != 2 || vocab % 8 != 0 || vocab > kRingMaxVocab || !aligned16(logits) || !aligned16(grad)) return 0;
    const std::size_t pitch = (static_cast<std::size_t>(vocab) * sizeof(T) + 127) / 128 * 128;
    std::size_t stages = kRingSmemBudget / pitch;
    if (stages > kRingMaxStages) stages = kRingMaxStages;
    if (stages < 2) return 0;
    *row_pitch = static_cast<unsigned>(pitch);
    return static_cast<int>(stages);
}

template <typename T>
int ce_ring_launch(float* row_loss, void* grad, const void* logits, const std::uint32_t* targets, long long rows, long long vocab,
                   float inv_total_rows, float gradient_scale, int stages, unsigned row_pitch, cudaStream_t s) {
    const std::size_t smem = static_cast<std::size_t>(stages) * row_pitch;
    static PerDeviceOnce attr_once;
    if (attr_once.needed()) {
        CGPT_CUDA_TRY(cudaFuncSetAttribute(cross_entropy_ring_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(kRingSmemBudget)));
        attr_once.done();
    }
    unsigned int* status = tc_status_device_ptr();
    if (status == nullptr) return CGPT_ERR_STATE;
    const unsigned grid = static_cast<unsigned>(rows < kNumSMs ? rows : kNumSMs);
    cross_entropy_ring_kernel<T><<<grid, kRingThreads, smem, s>>>(row_loss, static_cast<T*>(grad), static_cast<const T*>(logits), targets,
                                                                  rows, static_cast<int>(vocab), inv_total_rows, gradient_scale, stages,
                                                                  row_pitch, status);
    count_launch();
    CGPT_LAUNCH_CHECK();
    return CGPT_OK;
}

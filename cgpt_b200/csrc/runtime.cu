// Library-wide host state: version string, launch counter, per-device scratch arena.
#include <atomic>
#include <cstdlib>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "launch_counter.h"

namespace cgpt {

std::atomic<std::uint64_t> g_launch_count{0};

namespace {
constexpr int kMaxDevices = 64;
struct Arena {
    void* ptr = nullptr;
    std::size_t bytes = 0;
};
constexpr int kLanes = 2;                     // 0: the caller's stream, 1: the library's side stream
Arena g_arena[kMaxDevices][kLanes];
std::mutex g_arena_mutex;
thread_local std::size_t t_frame_offset = 0;  // bytes of the arena held by enclosing ScratchFrames
thread_local int t_lane = 0;                  // which arena ops issued by this thread use right now

struct Side {
    cudaStream_t stream = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
};
Side g_side[kMaxDevices];
std::atomic<int> g_branch_streams{-1};        // -1: not decided yet (environment), 0: off, 1: on
}  // namespace

// One arena per device and lane, shared by every op issued on that lane. Ops on one stream are ordered, so reuse
// is safe there. The block forward/backward run their two independent branches on two streams; whatever they issue
// on the side stream is issued inside a ScratchLane(1) scope and takes its scratch from the second arena, so the
// two streams never share scratch. Leaf ops take [offset, offset + bytes) where offset is the space held
// by enclosing ScratchFrames of the calling thread. Growth frees the old block with cudaFree (which
// synchronises the device, so earlier users have finished); it is refused while the stream is capturing
// and while a frame is open, because either would leave dangling pointers.
int scratch_get(void** out, std::size_t bytes, cudaStream_t stream) {
    int device = 0;
    CGPT_CUDA_TRY(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) return CGPT_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_arena_mutex);
    Arena& a = g_arena[device][t_lane];
    const std::size_t need = t_frame_offset + bytes;
    if (a.bytes < need) {
        if (t_frame_offset != 0) return CGPT_ERR_STATE;
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(stream, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone)
            return CGPT_ERR_STATE;
        std::size_t want = need < (std::size_t{64} << 20) ? (std::size_t{64} << 20) : need;
        want = (want + (std::size_t{1} << 20) - 1) & ~((std::size_t{1} << 20) - 1);
        if (a.ptr != nullptr) {
            CGPT_CUDA_TRY(cudaFree(a.ptr));
            a.ptr = nullptr;
            a.bytes = 0;
        }
        CGPT_CUDA_TRY(cudaMalloc(&a.ptr, want));
        a.bytes = want;
    }
    *out = static_cast<unsigned char*>(a.ptr) + t_frame_offset;
    return CGPT_OK;
}

ScratchFrame::ScratchFrame(std::size_t bytes, std::size_t inner_headroom, cudaStream_t stream) {
    held_ = (bytes + 1023) & ~std::size_t{1023};
    status = scratch_get(&ptr, held_ + inner_headroom, stream);
    if (status == CGPT_OK) t_frame_offset += held_;
    else held_ = 0;
}
ScratchFrame::~ScratchFrame() { t_frame_offset -= held_; }

ScratchLane::ScratchLane(int lane) : previous_(t_lane) { t_lane = lane; }
ScratchLane::~ScratchLane() { t_lane = previous_; }

int resident_ctas_per_sm(const void* kernel, int threads, std::size_t dynamic_smem) {
    struct Entry { const void* kernel; int device, threads; std::size_t smem; int ctas; };
    static std::mutex mutex;
    static std::vector<Entry> cache;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return 1;
    std::lock_guard<std::mutex> lock(mutex);
    for (const Entry& e : cache)
        if (e.kernel == kernel && e.device == device && e.threads == threads && e.smem == dynamic_smem) return e.ctas;
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, dynamic_smem) != cudaSuccess || n < 1) {
        cudaGetLastError();
        n = 1;
    }
    cache.push_back(Entry{kernel, device, threads, dynamic_smem, n});
    return n;
}

bool branch_streams_enabled() {
    int v = g_branch_streams.load(std::memory_order_relaxed);
    if (v < 0) {
        // Off unless asked for: at the 104m bench shape the step is power-capped and two streams gained 0.3-0.6 %.
        const char* e = std::getenv("CGPT_B200_BRANCH_STREAMS");
        v = (e != nullptr && e[0] == '1') ? 1 : 0;
        g_branch_streams.store(v, std::memory_order_relaxed);
    }
    return v == 1;
}

// The side stream and its two events, created on first use on a device. Creation is refused while `main` is being
// captured (the eager warm-up that precedes every capture creates them).
int side_stream_get(cudaStream_t main, cudaStream_t* side, cudaEvent_t* fork, cudaEvent_t* join) {
    int device = 0;
    CGPT_CUDA_TRY(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) return CGPT_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_arena_mutex);
    Side& sd = g_side[device];
    if (sd.stream == nullptr) {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(main, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone) return CGPT_ERR_STATE;
        CGPT_CUDA_TRY(cudaStreamCreateWithFlags(&sd.stream, cudaStreamNonBlocking));
        CGPT_CUDA_TRY(cudaEventCreateWithFlags(&sd.fork, cudaEventDisableTiming));
        CGPT_CUDA_TRY(cudaEventCreateWithFlags(&sd.join, cudaEventDisableTiming));
    }
    *side = sd.stream;
    *fork = sd.fork;
    *join = sd.join;
    return CGPT_OK;
}

}  // namespace cgpt

extern "C" int cgpt_b200_reserve_scratch(size_t bytes) {
    void* p = nullptr;
    return cgpt::scratch_get(&p, bytes, nullptr);
}

extern "C" int cgpt_b200_set_branch_streams(int enable) {
    cgpt::g_branch_streams.store(enable ? 1 : 0, std::memory_order_relaxed);
    return CGPT_OK;
}

extern "C" const char* cgpt_b200_version(void) { return "cgpt_b200 0.1 (sm_100a)"; }
extern "C" uint64_t cgpt_b200_launch_count(void) {
    return cgpt::g_launch_count.load(std::memory_order_relaxed);
}

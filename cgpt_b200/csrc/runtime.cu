// Library-wide host state: version string, launch counter, per-device scratch arena.
#include <mutex>

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
Arena g_arena[kMaxDevices];
std::mutex g_arena_mutex;
thread_local std::size_t t_frame_offset = 0;  // bytes of the arena held by enclosing ScratchFrames
}  // namespace

// One arena per device, shared by every op on that device. Ops on one stream are ordered, so reuse
// is safe there; ops issued concurrently on different streams of the same device must not rely on it
// (none of the training path does). Leaf ops take [offset, offset + bytes) where offset is the space held
// by enclosing ScratchFrames of the calling thread. Growth frees the old block with cudaFree (which
// synchronises the device, so earlier users have finished); it is refused while the stream is capturing
// and while a frame is open, because either would leave dangling pointers.
int scratch_get(void** out, std::size_t bytes, cudaStream_t stream) {
    int device = 0;
    CGPT_CUDA_TRY(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) return CGPT_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_arena_mutex);
    Arena& a = g_arena[device];
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

}  // namespace cgpt

extern "C" int cgpt_b200_reserve_scratch(size_t bytes) {
    void* p = nullptr;
    return cgpt::scratch_get(&p, bytes, nullptr);
}

extern "C" const char* cgpt_b200_version(void) { return "cgpt_b200 0.1 (sm_100a)"; }
extern "C" uint64_t cgpt_b200_launch_count(void) {
    return cgpt::g_launch_count.load(std::memory_order_relaxed);
}

// Device memory, streams and events behind the C ABI: the backend owns these itself, so a host that binds this
// library needs no other CUDA framework to run a plan.
//
//  * Region: ONE reservation of device memory per region (cudaMalloc on first use), blocks handed out first-fit at a
//    caller-chosen alignment (256 bytes by default) and coalesced with their free neighbours when given back. The
//    counterpart of the reference's region allocator (lumen/allocator/region.rs:13-121, lumen/allocator/cuda.rs:
//    59-121): allocation after the reservation is pure host bookkeeping - no driver call, nothing that a CUDA graph
//    capture could trip over. While a recorded graph launches into the region's blocks the region can be put on
//    HOLD: blocks freed meanwhile return only when the hold is released (cuda.rs:123-170 keeps such blocks per graph).
//  * Streams and events (lumen/runtime/stream/cuda.rs:119-290): thin owners of cudaStream_t / cudaEvent_t.
//  * Pinned host buffers and asynchronous copies for the step's inputs and results.
#include <algorithm>
#include <map>
#include <mutex>
#include <vector>

#include "device.h"

struct lb_region {
    int device = 0;
    size_t capacity = 0;
    char* base = nullptr;  // reserved on first take
    std::mutex mutex;
    std::map<size_t, size_t> free_blocks;  // offset -> bytes
    std::map<size_t, size_t> live;         // offset -> bytes
    size_t live_bytes = 0, peak_bytes = 0;
    int holds = 0;
    std::vector<std::pair<size_t, size_t>> held;  // blocks freed while on hold
};

namespace lb {
namespace {

constexpr size_t kAlign = 256;

void give_locked(lb_region& r, size_t offset, size_t bytes) {
    auto next = r.free_blocks.lower_bound(offset);
    if (next != r.free_blocks.begin()) {
        auto prev = std::prev(next);
        if (prev->first + prev->second == offset) {
            offset = prev->first;
            bytes += prev->second;
            r.free_blocks.erase(prev);
        }
    }
    if (next != r.free_blocks.end() && offset + bytes == next->first) {
        bytes += next->second;
        r.free_blocks.erase(next);
    }
    r.free_blocks[offset] = bytes;
}

}  // namespace
}  // namespace lb

extern "C" {

int lb_set_device(int device) {
    return lb::guarded([&] {
        lb::driver();
        LB_CUDA(cudaSetDevice(device));
        lb::device_info();  // refuses anything but sm_100
    });
}

int lb_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

int lb_device_synchronize(void) {
    return lb::guarded([&] { LB_CUDA(cudaDeviceSynchronize()); });
}

int lb_device_memory(size_t* free_bytes, size_t* total_bytes) {
    return lb::guarded([&] {
        size_t f = 0, t = 0;
        LB_CUDA(cudaMemGetInfo(&f, &t));
        if (free_bytes) *free_bytes = f;
        if (total_bytes) *total_bytes = t;
    });
}

int lb_region_create(size_t capacity_bytes, lb_region** out) {
    return lb::guarded([&] {
        if (!out || capacity_bytes == 0) lb::fail(LB_ERR_INVALID, "lb_region_create: a non-zero capacity and an out pointer");
        lb::driver();
        auto r = new lb_region;
        LB_CUDA(cudaGetDevice(&r->device));
        r->capacity = capacity_bytes - capacity_bytes % lb::kAlign;
        if (r->capacity == 0) {
            delete r;
            lb::fail(LB_ERR_INVALID, "lb_region_create: capacity below the 256-byte alignment");
        }
        r->free_blocks[0] = r->capacity;
        *out = r;
    });
}

void lb_region_destroy(lb_region* region) {
    if (!region) return;
    if (region->base) cudaFree(region->base);
    delete region;
}

int lb_region_alloc(lb_region* region, size_t bytes, size_t alignment, void** out) {
    return lb::guarded([&] {
        if (!region || !out) lb::fail(LB_ERR_INVALID, "lb_region_alloc: null argument");
        if (alignment == 0) alignment = lb::kAlign;
        if (alignment & (alignment - 1)) lb::fail(LB_ERR_INVALID, "lb_region_alloc: the alignment must be a power of two");
        alignment = std::max(alignment, lb::kAlign);
        const size_t want = std::max<size_t>((bytes + lb::kAlign - 1) / lb::kAlign * lb::kAlign, lb::kAlign);
        std::lock_guard<std::mutex> lock(region->mutex);
        if (!region->base) {  // the one reservation, with the region's device current
            int dev = 0;
            LB_CUDA(cudaGetDevice(&dev));
            if (dev != region->device) LB_CUDA(cudaSetDevice(region->device));
            cudaError_t err = cudaMalloc(&region->base, region->capacity);
            if (dev != region->device) cudaSetDevice(dev);
            if (err != cudaSuccess) {
                region->base = nullptr;
                lb::fail(LB_ERR_CUDA, lb::format("region: reserving %zu bytes on device %d failed: %s", region->capacity, region->device,
                                                 cudaGetErrorString(err)));
            }
        }
        const uintptr_t base = (uintptr_t)region->base;
        for (auto it = region->free_blocks.begin(); it != region->free_blocks.end(); ++it) {  // first fit, lowest offset
            const size_t offset = it->first, size = it->second;
            const size_t at = (size_t)(((base + offset + alignment - 1) & ~(uintptr_t)(alignment - 1)) - base);
            if (at + want > offset + size) continue;
            region->free_blocks.erase(it);
            if (at > offset) region->free_blocks[offset] = at - offset;
            if (at + want < offset + size) region->free_blocks[at + want] = offset + size - at - want;
            region->live[at] = want;
            region->live_bytes += want;
            region->peak_bytes = std::max(region->peak_bytes, region->live_bytes);
            *out = region->base + at;
            return;
        }
        size_t free_total = 0, largest = 0;
        for (auto& b : region->free_blocks) free_total += b.second, largest = std::max(largest, b.second);
        lb::fail(LB_ERR_CUDA, lb::format("region out of memory: %zu bytes requested, %zu of %zu bytes free (largest block %zu); create a "
                                         "larger region", bytes, free_total, region->capacity, largest));
    });
}

int lb_region_free(lb_region* region, void* ptr) {
    return lb::guarded([&] {
        if (!region) lb::fail(LB_ERR_INVALID, "lb_region_free: null region");
        if (!ptr) return;
        std::lock_guard<std::mutex> lock(region->mutex);
        const size_t offset = (size_t)((char*)ptr - region->base);
        auto it = region->base ? region->live.find(offset) : region->live.end();
        if (it == region->live.end()) lb::fail(LB_ERR_INVALID, "lb_region_free: the pointer is not a live block of this region");
        const size_t bytes = it->second;
        region->live.erase(it);
        region->live_bytes -= bytes;
        if (region->holds > 0) region->held.emplace_back(offset, bytes);  // a recorded graph may still launch into it
        else lb::give_locked(*region, offset, bytes);
    });
}

int lb_region_hold(lb_region* region) {
    return lb::guarded([&] {
        if (!region) lb::fail(LB_ERR_INVALID, "lb_region_hold: null region");
        std::lock_guard<std::mutex> lock(region->mutex);
        region->holds++;
    });
}

int lb_region_release(lb_region* region) {
    return lb::guarded([&] {
        if (!region) lb::fail(LB_ERR_INVALID, "lb_region_release: null region");
        std::lock_guard<std::mutex> lock(region->mutex);
        if (region->holds == 0) lb::fail(LB_ERR_INVALID, "lb_region_release: the region is not on hold");
        if (--region->holds == 0) {
            for (auto& b : region->held) lb::give_locked(*region, b.first, b.second);
            region->held.clear();
        }
    });
}

int lb_region_stats(lb_region* region, size_t* capacity, size_t* live_bytes, size_t* peak_bytes, size_t* largest_free) {
    return lb::guarded([&] {
        if (!region) lb::fail(LB_ERR_INVALID, "lb_region_stats: null region");
        std::lock_guard<std::mutex> lock(region->mutex);
        if (capacity) *capacity = region->capacity;
        if (live_bytes) *live_bytes = region->live_bytes;
        if (peak_bytes) *peak_bytes = region->peak_bytes;
        if (largest_free) {
            *largest_free = 0;
            for (auto& b : region->free_blocks) *largest_free = std::max(*largest_free, b.second);
        }
    });
}

// ---- streams and events ------------------------------------------------------------------------------------------
int lb_stream_create(void** out) {
    return lb::guarded([&] {
        if (!out) lb::fail(LB_ERR_INVALID, "lb_stream_create: null argument");
        lb::driver();
        cudaStream_t s = nullptr;
        LB_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
        *out = s;
    });
}
int lb_stream_destroy(void* stream) {
    return lb::guarded([&] {
        if (stream) LB_CUDA(cudaStreamDestroy((cudaStream_t)stream));
    });
}
int lb_stream_synchronize(void* stream) {
    return lb::guarded([&] { LB_CUDA(cudaStreamSynchronize((cudaStream_t)stream)); });
}
int lb_event_create(int timing, void** out) {
    return lb::guarded([&] {
        if (!out) lb::fail(LB_ERR_INVALID, "lb_event_create: null argument");
        lb::driver();
        cudaEvent_t e = nullptr;
        LB_CUDA(cudaEventCreateWithFlags(&e, timing ? cudaEventDefault : cudaEventDisableTiming));
        *out = e;
    });
}
int lb_event_destroy(void* event) {
    return lb::guarded([&] {
        if (event) LB_CUDA(cudaEventDestroy((cudaEvent_t)event));
    });
}
int lb_event_record(void* event, void* stream) {
    return lb::guarded([&] { LB_CUDA(cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream)); });
}
int lb_stream_wait_event(void* stream, void* event) {
    return lb::guarded([&] { LB_CUDA(cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)event, 0)); });
}
int lb_event_synchronize(void* event) {
    return lb::guarded([&] { LB_CUDA(cudaEventSynchronize((cudaEvent_t)event)); });
}
int lb_event_elapsed_ms(void* start, void* stop, float* ms) {
    return lb::guarded([&] {
        if (!ms) lb::fail(LB_ERR_INVALID, "lb_event_elapsed_ms: null argument");
        LB_CUDA(cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)stop));
    });
}

// ---- host memory and copies --------------------------------------------------------------------------------------
int lb_host_alloc(size_t bytes, void** out) {
    return lb::guarded([&] {
        if (!out) lb::fail(LB_ERR_INVALID, "lb_host_alloc: null argument");
        lb::driver();
        LB_CUDA(cudaHostAlloc(out, std::max<size_t>(bytes, 1), cudaHostAllocDefault));
    });
}
int lb_host_free(void* ptr) {
    return lb::guarded([&] {
        if (ptr) LB_CUDA(cudaFreeHost(ptr));
    });
}
int lb_copy_to_device(void* dst, const void* src, size_t bytes, void* stream) {
    return lb::guarded([&] { LB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream)); });
}
int lb_copy_to_host(void* dst, const void* src, size_t bytes, void* stream) {
    return lb::guarded([&] { LB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream)); });
}
int lb_copy_on_device(void* dst, const void* src, size_t bytes, void* stream) {
    return lb::guarded([&] { LB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream)); });
}
int lb_fill_bytes(void* dst, int byte, size_t bytes, void* stream) {
    return lb::guarded([&] { LB_CUDA(cudaMemsetAsync(dst, byte, bytes, (cudaStream_t)stream)); });
}
}

// Host-side runtime of the `paras` PrivateUse1 device for the B200 build.
//
// Keeps the reference's contract (csrc/core/context.h:34-74, csrc/core/allocator.h:34-73,
// csrc/core/registration.cpp:36-95): `paras:0` is the host, `paras:1..N` are the GPUs;
// the current device is thread-local; one stream per GPU; allocation happens on the
// current device; fork after first use is flagged.  Everything below it goes through the
// C ABI of libparas_b200 (include/paras_b200.h) -- this layer holds no CUDA call.
#pragma once

#include <ATen/ATen.h>
#include <c10/core/Allocator.h>
#include <c10/core/Device.h>

#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <mutex>
#include <vector>

#include "paras_b200.h"

namespace paras {

constexpr c10::DeviceType kDevice = c10::DeviceType::PrivateUse1;

// ---- logging: PTSYCL_LOG = 0 warnings, 1 device table + CPU fallbacks, 2 per-op trace
// (the reference's knob, csrc/core/log.h:30-60) ---------------------------------------
inline int log_level() {
    static const int lvl = [] {
        const char* e = std::getenv("PTSYCL_LOG");
        return e ? std::atoi(e) : 0;
    }();
    return lvl;
}
#define PARAS_INFO(...)                                    \
    do {                                                   \
        if (::paras::log_level() >= 1) {                   \
            std::fprintf(stderr, "[paras info] " __VA_ARGS__); \
            std::fprintf(stderr, "\n");                    \
        }                                                  \
    } while (0)
#define PARAS_TRACE_OP(name)                                              \
    do {                                                                  \
        if (::paras::log_level() >= 2) std::fprintf(stderr, "[paras op] %s\n", (name)); \
    } while (0)

// Turns a C-ABI status into the RuntimeError the reference's TORCH_CHECKs raise.
#define PARAS_ABI(call)                                                        \
    do {                                                                       \
        const int st_ = (call);                                                \
        TORCH_CHECK(st_ == PARAS_OK, paras_b200_last_error());                 \
    } while (0)

class Runtime {
public:
    static Runtime& get();

    int device_count() const { return 1 + gpu_count_; }  // host + GPUs
    int gpu_count() const { return gpu_count_; }
    bool is_gpu(int index) const { return index >= 1 && index <= gpu_count_; }
    // paras device index -> CUDA ordinal; raises for the host or a bad index
    int gpu_of(int index) const;
    int gpu_of(const at::Tensor& t) const { return gpu_of(int(t.device().index())); }
    void check_index(int index) const;
    std::string device_name(int index) const;

    void synchronize(int index);
    void synchronize_all();
    void empty_cache_all();
    uint64_t allocated_bytes(int index);
    uint64_t cached_bytes(int index);

    void set_seed(int index, uint64_t seed);
    void set_seed_all(uint64_t seed);
    // (seed, sequence) for an operator that draws `items` random numbers on device `index`, and the
    // sequence advanced as the reference's Context::rng_draw does (csrc/core/context.cpp:76-83: two
    // 32-bit values per Philox2x32 counter tick, plus one), so that a stream of random operators
    // sees the counters it would see there.  manual_seed resets the sequence to 0.
    std::pair<uint64_t, uint64_t> rng_draw(int index, int64_t items);

    static bool bad_fork();

    // raw memory on a paras device (host: 64-byte aligned malloc; GPU: stream-ordered pool)
    void* allocate(int index, size_t bytes);
    void release(int index, void* ptr, size_t bytes);

private:
    Runtime();
    int gpu_count_ = 0;
    std::atomic<uint64_t> host_bytes_{0};
    std::vector<uint64_t> seeds_;
    std::vector<uint64_t> sequences_;
    std::mutex rng_mu_;
};

c10::Allocator* device_allocator();
// A non-blocking host-to-GPU copy is about to read `ptr` on GPU ordinal `gpu`.  If `ptr` lies in
// a block of the cached pinned allocator, the block is not handed out again before that GPU's
// stream has drained (the freeing thread waits for it), so a later pin_memory() cannot
// overwrite bytes a queued DMA has yet to read.
void note_pinned_async_read(const void* ptr, int gpu);
// thread-local current device (csrc/core/registration.cpp:34)
c10::Device current_device();

inline int dtype_code(c10::ScalarType t) {
    switch (t) {
        case c10::kFloat: return PARAS_F32;
        case c10::kBFloat16: return PARAS_BF16;
        case c10::kHalf: return PARAS_F16;
        default: return -1;
    }
}

}  // namespace paras

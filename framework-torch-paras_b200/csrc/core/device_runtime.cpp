// Device table, allocator, device guard and hooks of the `paras` device (B200 build).
//
// Same contract as the reference's Context / ParasAllocator / ParasGuardImpl / ParasHooks
// (csrc/core/context.cpp:31-109, csrc/core/allocator.cpp:129-173,
// csrc/core/registration.cpp:36-95); the memory behind it is different: GPU tensors live in
// a stream-ordered cudaMallocAsync pool reached through the C ABI, never in unified memory,
// so nothing on the host may dereference a device pointer.
#include "core/device_runtime.h"

#include <ATen/detail/PrivateUse1HooksInterface.h>
#include <c10/core/impl/DeviceGuardImplInterface.h>
#include <pthread.h>
#include <torch/version.h>

#include <cstring>
#include <map>
#include <mutex>
#include <vector>

#if TORCH_VERSION_MAJOR < 2 || (TORCH_VERSION_MAJOR == 2 && TORCH_VERSION_MINOR < 4)
#error "the paras B200 backend requires PyTorch >= 2.4"
#endif

namespace paras {
namespace {

std::atomic<bool> g_initialised{false};
std::atomic<bool> g_bad_fork{false};

void on_fork_child() {
    if (g_initialised.load()) g_bad_fork.store(true);
}

thread_local c10::Device tl_device{kDevice, 0};

struct AllocRecord {
    void* ptr;
    int index;
    size_t bytes;
};

void delete_record(void* ctx) {
    auto* rec = static_cast<AllocRecord*>(ctx);
    if (!rec) return;
    // A tensor may be destroyed during interpreter shutdown; never throw from a deleter.
    try {
        Runtime::get().release(rec->index, rec->ptr, rec->bytes);
    } catch (...) {
    }
    delete rec;
}

class DeviceAllocator final : public c10::Allocator {
public:
    c10::DataPtr allocate(size_t nbytes) override {
        const c10::Device dev = tl_device;
        const int index = int(dev.index());
        if (nbytes == 0) return c10::DataPtr(nullptr, nullptr, &delete_record, dev);
        void* p = Runtime::get().allocate(index, nbytes);
        auto* rec = new AllocRecord{p, index, nbytes};
        return c10::DataPtr(p, rec, &delete_record, dev);
    }
    c10::DeleterFnPtr raw_deleter() const override { return nullptr; }
    void copy_data(void* dest, const void* src, std::size_t count) const override {
        const c10::Device dev = tl_device;
        Runtime& rt = Runtime::get();
        if (rt.is_gpu(int(dev.index()))) {
            PARAS_ABI(paras_b200_memcpy_d2d(rt.gpu_of(int(dev.index())), dest, src, count, nullptr));
        } else {
            std::memcpy(dest, src, count);
        }
    }
};

DeviceAllocator g_allocator;

// A device without an index means "the current one".
c10::Device with_index(c10::Device d) {
    return d.has_index() ? d : c10::Device(kDevice, tl_device.index());
}

struct GuardImpl final : public c10::impl::DeviceGuardImplInterface {
    c10::DeviceType type() const override { return kDevice; }
    c10::Device exchangeDevice(c10::Device d) const override {
        const c10::Device prev = tl_device;
        tl_device = with_index(d);
        return prev;
    }
    c10::Device getDevice() const override { return tl_device; }
    void setDevice(c10::Device d) const override { tl_device = with_index(d); }
    void uncheckedSetDevice(c10::Device d) const noexcept override { tl_device = with_index(d); }
    // One in-order queue per device, exposed as stream id 0.
    c10::Stream getStream(c10::Device d) const noexcept override {
        return c10::Stream(c10::Stream::UNSAFE, d, 0);
    }
    c10::Stream getDefaultStream(c10::Device d) const override { return getStream(d); }
    c10::Stream exchangeStream(c10::Stream) const noexcept override { return getStream(tl_device); }
    c10::DeviceIndex deviceCount() const noexcept override {
        try {
            return static_cast<c10::DeviceIndex>(Runtime::get().device_count());
        } catch (...) {
            return 0;
        }
    }
    bool queryStream(const c10::Stream&) const override { return true; }
    void synchronizeStream(const c10::Stream& s) const override {
        Runtime::get().synchronize(int(s.device().index()));
    }
    void synchronizeDevice(const c10::DeviceIndex index) const override {
        Runtime::get().synchronize(int(index));
    }
};

GuardImpl g_guard;
c10::impl::DeviceGuardImplRegistrar g_guard_registrar(kDevice, &g_guard);

// Page-locked host memory (`tensor.pin_memory()`, `torch.empty(..., pin_memory=True)`, and the
// destination of every device->host `.cpu()` copy): the source/destination of direct DMA
// transfers.  Pinning pages costs tens of milliseconds per 100 MB, so freed blocks are kept
// in size classes and handed out again; `empty_cache()` returns them to the system.
class PinnedCache {
public:
    void* take(size_t nbytes, size_t* rounded) {
        const size_t cls = round_up(nbytes);
        *rounded = cls;
        {
            std::lock_guard<std::mutex> lk(mu_);
            auto it = free_.find(cls);
            if (it != free_.end() && !it->second.empty()) {
                void* p = it->second.back();
                it->second.pop_back();
                cached_ -= cls;
                return p;
            }
        }
        void* p = nullptr;
        PARAS_ABI(paras_b200_host_alloc(cls, &p));
        return p;
    }
    // blocks in use, for note_async_read(): start address -> size class
    void track(void* p, size_t cls) {
        std::lock_guard<std::mutex> lk(mu_);
        live_[p] = cls;
    }
    void note_async_read(const void* ptr, int gpu) {
        if (gpu < 0 || gpu >= 64) return;
        std::lock_guard<std::mutex> lk(mu_);
        auto it = live_.upper_bound(const_cast<void*>(ptr));
        if (it == live_.begin()) return;
        --it;
        const char* base = static_cast<const char*>(it->first);
        if (static_cast<const char*>(ptr) < base + it->second) in_flight_[it->first] |= uint64_t(1) << gpu;
    }
    void give(void* p, size_t cls) {
        uint64_t gpus = 0;
        {
            std::lock_guard<std::mutex> lk(mu_);
            live_.erase(p);
            auto it = in_flight_.find(p);
            if (it != in_flight_.end()) {
                gpus = it->second;
                in_flight_.erase(it);
            }
        }
        // queued non-blocking copies may still have to read the block: let them finish first
        for (int g = 0; gpus; ++g, gpus >>= 1)
            if (gpus & 1) paras_b200_synchronize(g);
        std::lock_guard<std::mutex> lk(mu_);
        free_[cls].push_back(p);
        cached_ += cls;
    }
    void clear() {
        std::lock_guard<std::mutex> lk(mu_);
        for (auto& kv : free_)
            for (void* p : kv.second) paras_b200_host_free(p);
        free_.clear();
        cached_ = 0;
    }
    static PinnedCache& get() {
        static PinnedCache* c = new PinnedCache();  // leaked on purpose: tensors may outlive statics
        return *c;
    }

private:
    static size_t round_up(size_t n) {
        if (n <= 4096) return 4096;
        if (n <= (size_t(1) << 20)) {  // powers of two up to 1 MiB
            size_t c = 4096;
            while (c < n) c <<= 1;
            return c;
        }
        const size_t mb = size_t(2) << 20;  // then multiples of 2 MiB
        return (n + mb - 1) / mb * mb;
    }
    std::mutex mu_;
    std::map<size_t, std::vector<void*>> free_;
    std::map<void*, size_t> live_;
    std::map<void*, uint64_t> in_flight_;
    size_t cached_ = 0;
};

struct PinnedRecord {
    void* ptr;
    size_t cls;
};

void delete_pinned(void* ctx) {
    auto* rec = static_cast<PinnedRecord*>(ctx);
    if (!rec) return;
    PinnedCache::get().give(rec->ptr, rec->cls);
    delete rec;
}

class PinnedAllocator final : public c10::Allocator {
public:
    c10::DataPtr allocate(size_t nbytes) override {
        if (nbytes == 0) return c10::DataPtr(nullptr, nullptr, &delete_pinned, c10::Device(c10::kCPU));
        size_t cls = 0;
        void* p = PinnedCache::get().take(nbytes, &cls);
        PinnedCache::get().track(p, cls);
        return c10::DataPtr(p, new PinnedRecord{p, cls}, &delete_pinned, c10::Device(c10::kCPU));
    }
    c10::DeleterFnPtr raw_deleter() const override { return nullptr; }
    void copy_data(void* dest, const void* src, std::size_t count) const override {
        std::memcpy(dest, src, count);
    }
};

PinnedAllocator g_pinned_allocator;

struct Hooks final : public at::PrivateUse1HooksInterface {
    bool isBuilt() const override { return true; }
    bool isAvailable() const override { return Runtime::get().device_count() > 0; }
    bool hasPrimaryContext(c10::DeviceIndex index) const override {
        return index >= 0 && index < Runtime::get().device_count();
    }
    bool isPinnedPtr(const void* data) const override {
        return paras_b200_host_is_pinned(data) != 0;
    }
    c10::Allocator* getPinnedMemoryAllocator() const override { return &g_pinned_allocator; }
};

struct HooksRegistrar {
    Hooks hooks;
    HooksRegistrar() { at::RegisterPrivateUse1HooksInterface(&hooks); }
};
HooksRegistrar g_hooks_registrar;

}  // namespace

REGISTER_ALLOCATOR(kDevice, &g_allocator);

c10::Allocator* device_allocator() { return &g_allocator; }
void note_pinned_async_read(const void* ptr, int gpu) { PinnedCache::get().note_async_read(ptr, gpu); }
c10::Device current_device() { return tl_device; }

Runtime::Runtime() {
    gpu_count_ = paras_b200_device_count();
    seeds_.assign(size_t(1 + gpu_count_), 0x5deece66dULL);
    sequences_.assign(size_t(1 + gpu_count_), 0);
    static std::once_flag once;
    std::call_once(once, [] { pthread_atfork(nullptr, nullptr, &on_fork_child); });
    g_initialised.store(true);
    if (log_level() >= 1) {
        PARAS_INFO("backend %s: device 0 = host, %d GPU(s)", paras_b200_backend_name(), gpu_count_);
        for (int i = 1; i <= gpu_count_; ++i) PARAS_INFO("  paras:%d = %s", i, device_name(i).c_str());
    }
}

Runtime& Runtime::get() {
    static Runtime rt;
    return rt;
}

bool Runtime::bad_fork() { return g_bad_fork.load(); }

void Runtime::check_index(int index) const {
    TORCH_CHECK(index >= 0 && index < device_count(), "paras: invalid device index ", index,
                " (", device_count(), " device(s) available)");
}

int Runtime::gpu_of(int index) const {
    check_index(index);
    TORCH_CHECK(index >= 1,
                "paras: device 0 is the host; the B200 build runs this operator on paras:1.."
                " only and has no CPU fallback for it");
    return index - 1;
}

std::string Runtime::device_name(int index) const {
    check_index(index);
    if (index == 0) return "host";
    char buf[256];
    PARAS_ABI(paras_b200_device_name(index - 1, buf, sizeof(buf)));
    return buf;
}

void Runtime::synchronize(int index) {
    check_index(index);
    if (index >= 1) PARAS_ABI(paras_b200_synchronize(index - 1));
}

void Runtime::synchronize_all() {
    for (int i = 1; i <= gpu_count_; ++i) synchronize(i);
}

void Runtime::empty_cache_all() {
    for (int i = 0; i < gpu_count_; ++i) PARAS_ABI(paras_b200_pool_trim(i));
    PinnedCache::get().clear();
}

uint64_t Runtime::allocated_bytes(int index) {
    check_index(index);
    if (index == 0) return host_bytes_.load();
    uint64_t used = 0, reserved = 0;
    PARAS_ABI(paras_b200_pool_stats(index - 1, &used, &reserved));
    return used;
}

uint64_t Runtime::cached_bytes(int index) {
    check_index(index);
    if (index == 0) return 0;
    uint64_t used = 0, reserved = 0;
    PARAS_ABI(paras_b200_pool_stats(index - 1, &used, &reserved));
    return reserved > used ? reserved - used : 0;
}

void Runtime::set_seed(int index, uint64_t seed) {
    check_index(index);
    std::lock_guard<std::mutex> lk(rng_mu_);
    seeds_[size_t(index)] = seed;
    sequences_[size_t(index)] = 0;
}

void Runtime::set_seed_all(uint64_t seed) {
    std::lock_guard<std::mutex> lk(rng_mu_);
    for (auto& s : seeds_) s = seed;
    for (auto& q : sequences_) q = 0;
}

std::pair<uint64_t, uint64_t> Runtime::rng_draw(int index, int64_t items) {
    check_index(index);
    std::lock_guard<std::mutex> lk(rng_mu_);
    const uint64_t seq = sequences_[size_t(index)];
    sequences_[size_t(index)] += uint64_t((items + 1) / 2) + 1;
    return {seeds_[size_t(index)], seq};
}

void* Runtime::allocate(int index, size_t bytes) {
    check_index(index);
    if (index == 0) {
        void* p = nullptr;
        const size_t rounded = (bytes + 63) & ~size_t(63);
        TORCH_CHECK(posix_memalign(&p, 64, rounded) == 0, "paras: host allocation of ", bytes,
                    " bytes failed");
        host_bytes_ += bytes;
        return p;
    }
    void* p = nullptr;
    PARAS_ABI(paras_b200_malloc_async(index - 1, bytes, nullptr, &p));
    return p;
}

void Runtime::release(int index, void* ptr, size_t bytes) {
    if (!ptr) return;
    if (index == 0) {
        std::free(ptr);
        host_bytes_ -= bytes;
        return;
    }
    // Stream-ordered: the block returns to the pool once everything queued so far has run.
    paras_b200_free_async(index - 1, ptr, nullptr);
}

}  // namespace paras

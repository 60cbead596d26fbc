// Runtime half of the C ABI: device table, per-GPU stream, stream-ordered memory pool,
// host<->device copies through pinned staging.  Replaces the reference's compat layer
// (csrc/compat/paras_compat.cpp: enumerate_devices 87-135, Queue::init 230-254,
// Queue::alloc 270-307 [cudaMallocManaged], Queue::copy 326-352, Queue::synchronize) and
// the size-class MemoryPool of csrc/core/allocator.cpp with cudaMallocAsync on an
// explicit per-GPU pool: device memory is never host-addressable here, so unified-memory
// page faults cannot occur.
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <thread>
#include <vector>

#include <nvtx3/nvToolsExt.h>

#include "common.cuh"

namespace pb {

namespace {

thread_local char tl_error[1024] = "";
thread_local const char* tl_kernel = "";

struct Staging {
    std::mutex mu;
    static constexpr int kBufs = 4;
    static constexpr size_t kChunk = size_t(16) << 20;
    void* buf[kBufs] = {nullptr, nullptr, nullptr, nullptr};
    cudaEvent_t done[kBufs] = {nullptr, nullptr, nullptr, nullptr};
    bool ready = false;
};

struct Table {
    std::once_flag once;
    int count = 0;
    int init_status = PARAS_OK;
    std::vector<Gpu> gpus;
    std::vector<Staging*> staging;
};

Table& table() {
    static Table t;
    return t;
}

void init_table() {
    Table& t = table();
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
        cudaGetLastError();  // clear the sticky "no device" error
        n = 0;
    }
    t.gpus.resize(n);
    t.staging.resize(n, nullptr);
    for (int i = 0; i < n; ++i) {
        Gpu& g = t.gpus[i];
        g.ordinal = i;
        cudaDeviceProp p{};
        if (cudaGetDeviceProperties(&p, i) == cudaSuccess) {
            std::snprintf(g.name, sizeof(g.name), "%s", p.name);
            g.sm_count = p.multiProcessorCount;
            g.cc_major = p.major;
            g.cc_minor = p.minor;
            g.smem_optin = p.sharedMemPerBlockOptin;
        }
        t.staging[i] = new Staging();
    }
    t.count = n;
}

// PTSYCL_NO_CACHE / PTSYCL_DEBUG_ALLOC, the reference's allocator switches (csrc/core/allocator.cpp:
// 48-49): the first makes the pool hand freed memory back to the driver at the next synchronisation
// (release threshold 0) instead of caching it, for leak hunting; the second logs every allocation
// and release to stderr.
bool env_flag(const char* name) {
    const char* e = std::getenv(name);
    return e && *e && std::strcmp(e, "0") != 0;
}
bool debug_alloc() {
    static const bool on = env_flag("PTSYCL_DEBUG_ALLOC");
    return on;
}

// Streams and pools are created the first time a GPU is used, so that a process that
// only touches one GPU (one rank per GPU) creates no context on the others.
std::mutex g_lazy_mu;

int lazy_init_gpu(Gpu& g) {
    std::lock_guard<std::mutex> lk(g_lazy_mu);
    if (g.stream) return PARAS_OK;
    PB_CUDA(cudaSetDevice(g.ordinal));
    cudaStream_t s = nullptr, c = nullptr;
    PB_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    PB_CUDA(cudaStreamCreateWithFlags(&c, cudaStreamNonBlocking));
    cudaMemPoolProps props{};
    props.allocType = cudaMemAllocationTypePinned;
    props.handleTypes = cudaMemHandleTypeNone;
    props.location.type = cudaMemLocationTypeDevice;
    props.location.id = g.ordinal;
    cudaMemPool_t pool = nullptr;
    PB_CUDA(cudaMemPoolCreate(&pool, &props));
    // never trim on sync (180 GB of HBM is there to be cached) unless caching is switched off
    uint64_t keep = env_flag("PTSYCL_NO_CACHE") ? 0 : ~uint64_t(0);
    PB_CUDA(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep));
    int* hs = nullptr;
    int* ds = nullptr;
    PB_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&hs), sizeof(int), cudaHostAllocMapped));
    *hs = 0;
    PB_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void**>(&ds), hs, 0));
    g.status_host = hs;
    g.status_dev = ds;
    if (const char* lim = std::getenv("PARAS_POOL_LIMIT_MB")) g.limit_bytes = size_t(std::strtoull(lim, nullptr, 10)) << 20;
    g.pool = pool;
    g.copy_stream = c;
    g.stream = s;
    return PARAS_OK;
}

int ensure_staging(Gpu* g, Staging* st) {
    if (st->ready) return PARAS_OK;
    for (int i = 0; i < Staging::kBufs; ++i) {
        PB_CUDA(cudaHostAlloc(&st->buf[i], Staging::kChunk, cudaHostAllocDefault));
        PB_CUDA(cudaEventCreateWithFlags(&st->done[i], cudaEventDisableTiming));
    }
    (void)g;
    st->ready = true;
    return PARAS_OK;
}


// memcpy split over a few host threads: one core moves ~10 GB/s, PCIe Gen5 takes ~50.
void parallel_memcpy(void* dst, const void* src, size_t bytes) {
    constexpr size_t kMinPerThread = size_t(2) << 20;
    unsigned hw = std::thread::hardware_concurrency();
    size_t nthreads = bytes / kMinPerThread;
    if (nthreads > 4) nthreads = 4;
    if (hw && nthreads > hw) nthreads = hw;
    if (nthreads <= 1) {
        std::memcpy(dst, src, bytes);
        return;
    }
    size_t per = (bytes / nthreads + 63) & ~size_t(63);
    std::vector<std::thread> th;
    for (size_t i = 1; i < nthreads; ++i) {
        size_t off = i * per;
        if (off >= bytes) break;
        size_t len = (off + per > bytes) ? bytes - off : per;
        th.emplace_back([=] {
            std::memcpy(static_cast<char*>(dst) + off, static_cast<const char*>(src) + off, len);
        });
    }
    std::memcpy(dst, src, per < bytes ? per : bytes);
    for (auto& t : th) t.join();
}

}  // namespace

NvtxRange::NvtxRange(const char* name) {
    static const bool enabled = std::getenv("PARAS_NVTX") != nullptr;
    on = enabled;
    if (on) nvtxRangePushA(name);
}
NvtxRange::~NvtxRange() {
    if (on) nvtxRangePop();
}

bool host_ptr_is_pinned(const void* p) {
    cudaPointerAttributes a{};
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return a.type == cudaMemoryTypeHost;
}

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    std::vsnprintf(tl_error, sizeof(tl_error), fmt, ap);
    va_end(ap);
    return code;
}

void set_last_kernel(const char* name) { tl_kernel = name; }

int check_status_word(Gpu* g) {
    if (!g || !g->status_host) return PARAS_OK;
    const int code = *static_cast<volatile int*>(g->status_host);
    if (code == 0) return PARAS_OK;
    *static_cast<volatile int*>(g->status_host) = 0;
    return fail(PARAS_E_TIMEOUT,
                "paras_b200: a kernel on gpu %d gave up a bounded wait (status word %d); its "
                "output is invalid", g->ordinal, code);
}

Gpu* use_gpu(int gpu, int* status) {
    Table& t = table();
    std::call_once(t.once, init_table);
    if (t.count == 0) {
        *status = fail(PARAS_E_NODEVICE,
                       "paras_b200: no CUDA GPU is visible; this build has no CPU fallback");
        return nullptr;
    }
    if (gpu < 0 || gpu >= t.count) {
        *status = fail(PARAS_E_INVALID, "paras_b200: gpu ordinal %d out of range [0,%d)", gpu,
                       t.count);
        return nullptr;
    }
    Gpu& g = t.gpus[gpu];
    if (!g.stream) {
        int s = lazy_init_gpu(g);
        if (s != PARAS_OK) {
            *status = s;
            return nullptr;
        }
    }
    cudaError_t e = cudaSetDevice(gpu);
    if (e != cudaSuccess) {
        *status = fail(PARAS_E_CUDA, "paras_b200: cudaSetDevice(%d): %s", gpu,
                       cudaGetErrorString(e));
        return nullptr;
    }
    *status = PARAS_OK;
    return &g;
}

}  // namespace pb

using pb::fail;
using pb::Gpu;
using pb::use_gpu;

extern "C" {

int paras_b200_abi_version(void) { return PARAS_B200_ABI_VERSION; }

const char* paras_b200_backend_name(void) { return "paras-b200-sm100a"; }

const char* paras_b200_last_error(void) { return pb::tl_error; }

const char* paras_b200_sdpa_last_kernel(void) { return pb::tl_kernel; }

int paras_b200_device_count(void) {
    pb::Table& t = pb::table();
    std::call_once(t.once, pb::init_table);
    return t.count;
}

int paras_b200_device_name(int gpu, char* buf, size_t buflen) {
    pb::Table& t = pb::table();
    std::call_once(t.once, pb::init_table);
    if (!buf || buflen == 0) return fail(PARAS_E_INVALID, "paras_b200: null name buffer");
    if (gpu < 0 || gpu >= t.count)
        return fail(t.count ? PARAS_E_INVALID : PARAS_E_NODEVICE,
                    "paras_b200: gpu ordinal %d out of range [0,%d)", gpu, t.count);
    std::snprintf(buf, buflen, "%s", t.gpus[gpu].name);
    return PARAS_OK;
}

int paras_b200_device_sm_count(int gpu, int* sms) {
    pb::Table& t = pb::table();
    std::call_once(t.once, pb::init_table);
    if (!sms) return fail(PARAS_E_INVALID, "paras_b200: null output");
    if (gpu < 0 || gpu >= t.count)
        return fail(t.count ? PARAS_E_INVALID : PARAS_E_NODEVICE,
                    "paras_b200: gpu ordinal %d out of range [0,%d)", gpu, t.count);
    *sms = t.gpus[gpu].sm_count;
    return PARAS_OK;
}

int paras_b200_stream(int gpu, void** stream) {
    if (!stream) return fail(PARAS_E_INVALID, "paras_b200: null output");
    int st;
    Gpu* g = use_gpu(gpu, &st);
    if (!g) return st;
    *stream = g->stream;
    return PARAS_OK;
}

int paras_b200_synchronize(int gpu) {
    int st;
    Gpu* g = use_gpu(gpu, &st);
    if (!g) return st;
    PB_CUDA(cudaStreamSynchronize(g->stream));
    return pb::check_status_word(g);
}

int paras_b200_pool_set_limit(int gpu, size_t bytes) {
    int st;
    Gpu* g = use_gpu(gpu, &st);
    if (!g) return st;
    g->limit_bytes = bytes;
    return PARAS_OK;
}

int paras_b200_malloc_async(int gpu, size_t bytes, void* stream, void** ptr) {
    pb::NvtxRange range("paras_b200_malloc_async");
    if (!ptr) return fail(PARAS_E_INVALID, "paras_b200: null output");
    *ptr = nullptr;
    int st;
    Gpu* g = use_gpu(gpu, &st);
    if (!g) return st;
    if (bytes == 0) return PARAS_OK;
    if (g->limit_bytes) {
        uint64_t used = 0;
        PB_CUDA(cudaMemPoolGetAttribute(g->pool, cudaMemPoolAttrUsedMemCurrent, &used));
        if (used + bytes > g->limit_bytes)
            return fail(PARAS_E_NOMEM, "paras_b200: out of memory on gpu %d: %zu bytes asked for with %llu in use and a "
                        "limit of %zu (paras_b200_pool_set_limit / PARAS_POOL_LIMIT_MB)", gpu, bytes,
                        static_cast<unsigned long long>(used), g->limit_bytes);
    }
    cudaError_t e = cudaMallocFromPoolAsync(ptr, bytes, g->pool, pb::pick_stream(g, stream));
    if (e == cudaErrorMemoryAllocation) {
        cudaGetLastError();
        // Give cached blocks back and retry once before reporting out-of-memory.
        cudaStreamSynchronize(pb::pick_stream(g, stream));
        cudaMemPoolTrimTo(g->pool, 0);
        e = cudaMallocFromPoolAsync(ptr, bytes, g->pool, pb::pick_stream(g, stream));
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        *ptr = nullptr;
        return fail(e == cudaErrorMemoryAllocation ? PARAS_E_NOMEM : PARAS_E_CUDA,
                    "paras_b200: cudaMallocFromPoolAsync(%zu bytes) on gpu %d: %s", bytes, gpu,
                    cudaGetErrorString(e));
    }
    if (pb::debug_alloc()) std::fprintf(stderr, "[paras_b200] gpu %d alloc %zu bytes -> %p\n", gpu, bytes, *ptr);
    return PARAS_OK;
}

int paras_b200_free_async(int gpu, void* ptr, void* stream) {
    if (!ptr) return PARAS_OK;
    int st;
    Gpu* g = use_gpu(gpu, &st);
    if (!g) return st;
    PB_CUDA(cudaFreeAsync(ptr, pb::pick_stream(g, stream)));
    if (pb::debug_alloc()) std::fprintf(stderr, "[paras_b200] gpu %d free %p\n", gpu, ptr);
    return PARAS_OK;
}

int paras_b200_pool_stats(int gpu, uint64_t* used_bytes, uint64_t* reserved_bytes) {
    int st;
    Gpu* g = use_gpu(gpu, &st);
    if (!g) return st;
    uint64_t used = 0, reserved = 0;
    PB_CUDA(cudaMemPoolGetAttribute(g->pool, cudaMemPoolAttrUsedMemCurrent, &used));
    PB_CUDA(cudaMemPoolGetAttribute(g->pool, cudaMemPoolAttrReservedMemCurrent, &reserved));
    if (used_bytes) *used_bytes = used;
    if (reserved_bytes) *reserved_bytes = reserved;
    return PARAS_OK;
}

int paras_b200_pool_trim(int gpu) {
    int st;
    Gpu* g = use_gpu(gpu, &st);
    if (!g) return st;
    PB_CUDA(cudaStreamSynchronize(g->stream));
    PB_CUDA(cudaMemPoolTrimTo(g->pool, 0));
    return PARAS_OK;
}

int paras_b200_memcpy_h2d(int gpu, void* dst, const void* src, size_t bytes, void* stream,
                          int blocking) {
    if (bytes == 0) return PARAS_OK;
    if (!dst || !src) return fail(PARAS_E_INVALID, "paras_b200: null pointer in memcpy_h2d");
    int st;
    Gpu* g = use_gpu(gpu, &st);
    if (!g) return st;
    cudaStream_t s = pb::pick_stream(g, stream);
    if (pb::host_ptr_is_pinned(src)) {
        PB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, s));
        if (blocking) PB_CUDA(cudaStreamSynchronize(s));
        return PARAS_OK;
    }
    // Pageable source: pipeline host memcpy -> pinned chunk -> DMA over a ring of chunks.
    pb::Staging* sg = pb::table().staging[gpu];
    std::lock_guard<std::mutex> lk(sg->mu);
    st = pb::ensure_staging(g, sg);
    if (st != PARAS_OK) return st;
    size_t off = 0;
    int i = 0;
    while (off < bytes) {
        size_t len = bytes - off < pb::Staging::kChunk ? bytes - off : pb::Staging::kChunk;
        PB_CUDA(cudaEventSynchronize(sg->done[i]));  // chunk i's previous DMA has drained
        pb::parallel_memcpy(sg->buf[i], static_cast<const char*>(src) + off, len);
        PB_CUDA(cudaMemcpyAsync(static_cast<char*>(dst) + off, sg->buf[i], len,
                                cudaMemcpyHostToDevice, s));
        PB_CUDA(cudaEventRecord(sg->done[i], s));
        off += len;
        i = (i + 1) % pb::Staging::kBufs;
    }
    if (blocking) PB_CUDA(cudaStreamSynchronize(s));
    return PARAS_OK;
}

int paras_b200_memcpy_d2h(int gpu, void* dst, const void* src, size_t bytes, void* stream) {
    if (bytes == 0) return PARAS_OK;
    if (!dst || !src) return fail(PARAS_E_INVALID, "paras_b200: null pointer in memcpy_d2h");
    int st;
    Gpu* g = use_gpu(gpu, &st);
    if (!g) return st;
    cudaStream_t s = pb::pick_stream(g, stream);
    if (pb::host_ptr_is_pinned(dst)) {
        PB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, s));
        PB_CUDA(cudaStreamSynchronize(s));
        return PARAS_OK;
    }
    pb::Staging* sg = pb::table().staging[gpu];
    std::lock_guard<std::mutex> lk(sg->mu);
    st = pb::ensure_staging(g, sg);
    if (st != PARAS_OK) return st;
    // Issue DMA for chunk c+1.. while the host drains chunk c.
    const size_t nchunks = (bytes + pb::Staging::kChunk - 1) / pb::Staging::kChunk;
    size_t issued = 0;
    for (size_t c = 0; c < nchunks; ++c) {
        while (issued < nchunks && issued < c + pb::Staging::kBufs) {
            size_t off = issued * pb::Staging::kChunk;
            size_t len = bytes - off < pb::Staging::kChunk ? bytes - off : pb::Staging::kChunk;
            int bi = int(issued % pb::Staging::kBufs);
            PB_CUDA(cudaMemcpyAsync(sg->buf[bi], static_cast<const char*>(src) + off, len,
                                    cudaMemcpyDeviceToHost, s));
            PB_CUDA(cudaEventRecord(sg->done[bi], s));
            ++issued;
        }
        size_t off = c * pb::Staging::kChunk;
        size_t len = bytes - off < pb::Staging::kChunk ? bytes - off : pb::Staging::kChunk;
        int bi = int(c % pb::Staging::kBufs);
        PB_CUDA(cudaEventSynchronize(sg->done[bi]));
        pb::parallel_memcpy(static_cast<char*>(dst) + off, sg->buf[bi], len);
    }
    return PARAS_OK;
}

int paras_b200_memcpy_d2d(int gpu, void* dst, const void* src, size_t bytes, void* stream) {
    if (bytes == 0) return PARAS_OK;
    if (!dst || !src) return fail(PARAS_E_INVALID, "paras_b200: null pointer in memcpy_d2d");
    int st;
    Gpu* g = use_gpu(gpu, &st);
    if (!g) return st;
    PB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, pb::pick_stream(g, stream)));
    return PARAS_OK;
}

int paras_b200_memcpy_peer(int dst_gpu, void* dst, int src_gpu, const void* src, size_t bytes) {
    if (bytes == 0) return PARAS_OK;
    if (!dst || !src) return fail(PARAS_E_INVALID, "paras_b200: null pointer in memcpy_peer");
    int st;
    Gpu* gs = use_gpu(src_gpu, &st);
    if (!gs) return st;
    PB_CUDA(cudaStreamSynchronize(gs->stream));  // source data is complete
    Gpu* gd = use_gpu(dst_gpu, &st);
    if (!gd) return st;
    PB_CUDA(cudaMemcpyPeerAsync(dst, dst_gpu, src, src_gpu, bytes, gd->stream));
    PB_CUDA(cudaStreamSynchronize(gd->stream));
    return PARAS_OK;
}

int paras_b200_memset(int gpu, void* dst, int value, size_t bytes, void* stream) {
    if (bytes == 0) return PARAS_OK;
    if (!dst) return fail(PARAS_E_INVALID, "paras_b200: null pointer in memset");
    int st;
    Gpu* g = use_gpu(gpu, &st);
    if (!g) return st;
    PB_CUDA(cudaMemsetAsync(dst, value, bytes, pb::pick_stream(g, stream)));
    return PARAS_OK;
}

int paras_b200_host_alloc(size_t bytes, void** ptr) {
    if (!ptr) return fail(PARAS_E_INVALID, "paras_b200: null output");
    *ptr = nullptr;
    if (paras_b200_device_count() == 0)
        return fail(PARAS_E_NODEVICE, "paras_b200: no CUDA GPU is visible");
    if (bytes == 0) return PARAS_OK;
    cudaError_t e = cudaHostAlloc(ptr, bytes, cudaHostAllocPortable);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(PARAS_E_NOMEM, "paras_b200: cudaHostAlloc(%zu): %s", bytes,
                    cudaGetErrorString(e));
    }
    return PARAS_OK;
}

int paras_b200_host_is_pinned(const void* ptr) {
    if (!ptr || paras_b200_device_count() == 0) return 0;
    return pb::host_ptr_is_pinned(ptr) ? 1 : 0;
}

int paras_b200_host_free(void* ptr) {
    if (!ptr) return PARAS_OK;
    PB_CUDA(cudaFreeHost(ptr));
    return PARAS_OK;
}

}  // extern "C"

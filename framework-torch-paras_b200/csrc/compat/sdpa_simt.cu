// General scaled-dot-product-attention forward on CUDA cores (fp32 accumulate, online
// softmax), plus the split-KV combine kernel.
//
// This is the path for what the tensor-core kernels do not take: fp32 tensors (the
// reference's own tests are fp32 with a 1e-4 tolerance, which TF32 tensor cores would not
// meet), head dims other than 128, explicit bool / additive masks
// (csrc/ops/attention_ops.cpp:117-126) and odd strides.  It never materialises the
// [B,H,Lq,Lk] score tensor that the reference's composition builds several times over
// (attention_ops.cpp:101-134).
//
// One warp per query row.  Each lane scores one key of a 32-key chunk (dot product over
// D with q broadcast from shared memory), the chunk's max/sum are warp reductions, and
// the P*V update gives lane l the output dims l, l+32, ... so V rows are read coalesced.
#include <cfloat>
#include <mutex>

#include "sdpa_common.cuh"

namespace pb {
namespace {

constexpr int kRowsPerBlock = 4;  // warps per CTA, one query row each
constexpr int kMaxD = 256;

struct SimtParams {
    const void* q;
    const void* k;
    const void* v;
    void* out;
    float* lse;
    const void* mask;
    int mask_kind;
    int B, Hq, Hkv, Lq, Lk, D;
    int64_t qs[3], ks[3], vs[3], os[3], ms[4];
    int causal;
    float scale;
    int splits;
    int keys_per_split;
    float* o_part;
    float2* ml_part;
};

template <typename T>
__global__ void __launch_bounds__(kRowsPerBlock * 32)
sdpa_simt_kernel(const SimtParams p) {
    __shared__ float sq[kRowsPerBlock][kMaxD];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qi = blockIdx.x * kRowsPerBlock + warp;
    const int h = blockIdx.y;
    const int b = blockIdx.z / p.splits;
    const int split = blockIdx.z - b * p.splits;
    const int hk = h / (p.Hq / p.Hkv);
    const int D = p.D;
    if (qi >= p.Lq) return;  // whole warp leaves; no block-wide barrier below

    const T* qrow = static_cast<const T*>(p.q) + b * p.qs[0] + h * p.qs[1] + int64_t(qi) * p.qs[2];
    for (int d = lane; d < D; d += 32) sq[warp][d] = to_f32<T>(qrow[d]);
    __syncwarp();

    int k_begin = split * p.keys_per_split;
    int k_end = min(p.Lk, k_begin + p.keys_per_split);
    if (p.causal) k_end = min(k_end, qi + 1);  // top-left aligned: keys 0..qi

    const T* kbase = static_cast<const T*>(p.k) + b * p.ks[0] + hk * p.ks[1];
    const T* vbase = static_cast<const T*>(p.v) + b * p.vs[0] + hk * p.vs[1];
    const bool kvec = (D % Vec16<T>::N == 0) && ((reinterpret_cast<uintptr_t>(kbase) & 15u) == 0) &&
                      ((p.ks[2] * int64_t(sizeof(T))) % 16 == 0);

    float acc[kMaxD / 32];
#pragma unroll
    for (int i = 0; i < kMaxD / 32; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;

    for (int k0 = k_begin; k0 < k_end; k0 += 32) {
        const int key = k0 + lane;
        float s = -INFINITY;
        if (key < k_end) {
            const T* krow = kbase + int64_t(key) * p.ks[2];
            float dot = 0.f;
            if (kvec) {
                constexpr int N = Vec16<T>::N;
                for (int d = 0; d < D; d += N) {
                    const Vec16<T> kv = ld16(krow + d);
#pragma unroll
                    for (int e = 0; e < N; ++e) dot = fmaf(sq[warp][d + e], to_f32<T>(kv.v[e]), dot);
                }
            } else {
                for (int d = 0; d < D; ++d) dot = fmaf(sq[warp][d], to_f32<T>(krow[d]), dot);
            }
            s = dot * p.scale;
            if (p.mask_kind) {
                const int64_t mo = b * p.ms[0] + h * p.ms[1] + int64_t(qi) * p.ms[2] + int64_t(key) * p.ms[3];
                if (p.mask_kind == 1) {
                    if (!static_cast<const unsigned char*>(p.mask)[mo]) s = -INFINITY;
                } else if (p.mask_kind == 2) {
                    s += to_f32<T>(static_cast<const T*>(p.mask)[mo]);
                } else {
                    s += static_cast<const float*>(p.mask)[mo];
                }
            }
        }
        const float cmax = warp_max(s);
        const float m_new = fmaxf(m, cmax);
        float pj = 0.f, alpha = 1.f;
        if (m_new != -INFINITY) {  // otherwise nothing attended yet: keep acc = 0, l = 0
            pj = (s == -INFINITY) ? 0.f : expf(s - m_new);
            alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
        }
        l = l * alpha + warp_sum(pj);
        m = m_new;
#pragma unroll
        for (int i = 0; i < kMaxD / 32; ++i) acc[i] *= alpha;
        const int valid = min(32, k_end - k0);
        for (int j = 0; j < valid; ++j) {
            const float pv = __shfl_sync(0xffffffffu, pj, j);
            const T* vrow = vbase + int64_t(k0 + j) * p.vs[2];
#pragma unroll
            for (int i = 0; i < kMaxD / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < D) acc[i] = fmaf(pv, to_f32<T>(vrow[d]), acc[i]);
            }
        }
    }

    const int64_t row = (int64_t(b) * p.Hq + h) * p.Lq + qi;
    if (p.splits > 1) {
        float* op = p.o_part + (int64_t(split) * (int64_t(p.B) * p.Hq * p.Lq) + row) * D;
#pragma unroll
        for (int i = 0; i < kMaxD / 32; ++i) {
            const int d = lane + 32 * i;
            if (d < D) op[d] = acc[i];
        }
        if (lane == 0) p.ml_part[int64_t(split) * (int64_t(p.B) * p.Hq * p.Lq) + row] = make_float2(m, l);
        return;
    }
    // l == 0 only when every key was masked out: the reference's softmax then yields NaN
    // (exp(-inf - -inf)); with no keys at all (Lk == 0) its matmul over an empty dim is 0.
    const float inv = 1.0f / l;
    T* orow = static_cast<T*>(p.out) + b * p.os[0] + h * p.os[1] + int64_t(qi) * p.os[2];
#pragma unroll
    for (int i = 0; i < kMaxD / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < D)
            orow[d] = from_f32<T>(l == 0.f ? (p.Lk == 0 ? 0.f : __int_as_float(0x7fc00000))
                                           : acc[i] * inv);
    }
    if (p.lse && lane == 0) p.lse[row] = (l == 0.f) ? -INFINITY : m + logf(l);
}

struct CombineParams {
    void* out;
    float* lse;
    int B, Hq, Lq, D;
    int64_t os[3];
    int splits;
    const float* o_part;
    const float2* ml_part;
};

// One warp per output row: weights exp(m_s - m) over the splits, then normalise.
template <typename T>
__global__ void __launch_bounds__(128)
sdpa_combine_kernel(const CombineParams p) {
    const int lane = threadIdx.x & 31;
    const int64_t rows = int64_t(p.B) * p.Hq * p.Lq;
    const int64_t row = int64_t(blockIdx.x) * 4 + (threadIdx.x >> 5);
    if (row >= rows) return;
    float m = -INFINITY;
    for (int s = 0; s < p.splits; ++s) m = fmaxf(m, p.ml_part[int64_t(s) * rows + row].x);
    float l = 0.f;
    for (int s = 0; s < p.splits; ++s) {
        const float2 ml = p.ml_part[int64_t(s) * rows + row];
        if (ml.x != -INFINITY) l += ml.y * expf(ml.x - m);
    }
    const int qi = int(row % p.Lq);
    const int h = int((row / p.Lq) % p.Hq);
    const int b = int(row / (int64_t(p.Lq) * p.Hq));
    T* orow = static_cast<T*>(p.out) + b * p.os[0] + h * p.os[1] + int64_t(qi) * p.os[2];
    const float inv = 1.0f / l;
    for (int d = lane; d < p.D; d += 32) {
        float acc = 0.f;
        for (int s = 0; s < p.splits; ++s) {
            const float2 ml = p.ml_part[int64_t(s) * rows + row];
            if (ml.x != -INFINITY)
                acc = fmaf(p.o_part[(int64_t(s) * rows + row) * p.D + d], expf(ml.x - m), acc);
        }
        orow[d] = from_f32<T>(l == 0.f ? __int_as_float(0x7fc00000) : acc * inv);
    }
    if (p.lse && lane == 0) p.lse[row] = (l == 0.f) ? -INFINITY : m + logf(l);
}

}  // namespace

int sdpa_simt_pick_splits(const Gpu* g, const paras_sdpa_args& a) {
    const int sms = g->sm_count > 0 ? g->sm_count : 148;
    const int64_t blocks = int64_t((a.Lq + kRowsPerBlock - 1) / kRowsPerBlock) * a.Hq * a.B;
    if (blocks >= int64_t(sms) * 4 || a.Lk < 1024) return 1;
    int64_t want = (int64_t(sms) * 8 + blocks - 1) / blocks;
    const int64_t max_by_len = a.Lk / 256;
    if (want > max_by_len) want = max_by_len;
    if (want > 64) want = 64;
    return want < 1 ? 1 : int(want);
}

int sdpa_simt_launch(Gpu* g, const paras_sdpa_args& a, float scale, const SplitWorkspace& ws,
                     cudaStream_t s) {
    if (a.D > kMaxD)
        return fail(PARAS_E_UNSUPPORTED, "paras sdpa: head dim %d exceeds kernel limit %d", a.D, kMaxD);
    if (int64_t(a.B) * ws.splits > 65535 || a.Hq > 65535)
        return fail(PARAS_E_UNSUPPORTED, "paras sdpa: batch*splits or heads exceed the grid limit");
    SimtParams p{};
    p.q = a.q; p.k = a.k; p.v = a.v; p.out = a.out; p.lse = a.lse;
    p.mask = a.mask; p.mask_kind = a.mask ? a.mask_kind : 0;
    p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv; p.Lq = a.Lq; p.Lk = a.Lk; p.D = a.D;
    for (int i = 0; i < 3; ++i) {
        p.qs[i] = a.q_strides[i]; p.ks[i] = a.k_strides[i];
        p.vs[i] = a.v_strides[i]; p.os[i] = a.o_strides[i];
    }
    for (int i = 0; i < 4; ++i) p.ms[i] = a.mask_strides[i];
    p.causal = a.causal;
    p.scale = scale;
    p.splits = ws.splits;
    p.keys_per_split = ws.splits > 1 ? ((a.Lk + ws.splits - 1) / ws.splits + 31) / 32 * 32 : a.Lk;
    p.o_part = ws.o_part;
    p.ml_part = ws.ml_part;
    dim3 grid((a.Lq + kRowsPerBlock - 1) / kRowsPerBlock, a.Hq, a.B * ws.splits);
    switch (a.dtype) {
        case PARAS_F32: sdpa_simt_kernel<float><<<grid, kRowsPerBlock * 32, 0, s>>>(p); break;
        case PARAS_BF16: sdpa_simt_kernel<__nv_bfloat16><<<grid, kRowsPerBlock * 32, 0, s>>>(p); break;
        default: sdpa_simt_kernel<__half><<<grid, kRowsPerBlock * 32, 0, s>>>(p); break;
    }
    PB_LAUNCH_CHECK("sdpa_simt_kernel");
    if (ws.splits > 1) return sdpa_combine_launch(g, a, ws, s);
    return PARAS_OK;
}

int sdpa_combine_launch(Gpu* g, const paras_sdpa_args& a, const SplitWorkspace& ws,
                        cudaStream_t s) {
    (void)g;
    CombineParams c{};
    c.out = a.out; c.lse = a.lse;
    c.B = a.B; c.Hq = a.Hq; c.Lq = a.Lq; c.D = a.D;
    for (int i = 0; i < 3; ++i) c.os[i] = a.o_strides[i];
    c.splits = ws.splits;
    c.o_part = ws.o_part;
    c.ml_part = ws.ml_part;
    const int64_t rows = int64_t(a.B) * a.Hq * a.Lq;
    const int64_t blocks = (rows + 3) / 4;
    switch (a.dtype) {
        case PARAS_F32: sdpa_combine_kernel<float><<<int(blocks), 128, 0, s>>>(c); break;
        case PARAS_BF16: sdpa_combine_kernel<__nv_bfloat16><<<int(blocks), 128, 0, s>>>(c); break;
        default: sdpa_combine_kernel<__half><<<int(blocks), 128, 0, s>>>(c); break;
    }
    PB_LAUNCH_CHECK("sdpa_combine_kernel");
    return PARAS_OK;
}

}  // namespace pb

// ---------------------------------------------------------------------------------------
// paras_b200_sdpa_fwd_static_scratch: the split-KV CUDA-core kernel above, with its partial
// results kept in a fixed array inside this library instead of allocated memory.
//
// Some callers cannot allocate device memory at the moment they need attention: a serving
// process whose own memory manager claimed the whole GPU at start-up (a cudaMalloc from
// inside a request then fails or stalls behind an implicit synchronisation), or a decode loop
// with a latency budget that has no room for an allocator call.  For them this entry point
// allocates nothing -- no cudaMalloc/cudaFree, no pool, no stream or event creation: the
// scratch is the file-scope device array below (held by every GPU that loads the library,
// until the process exits), the launch goes to the caller's stream.
//
// The array's name is only a host-side handle; its device address is looked up once per
// GPU, with that GPU current, by cudaGetSymbolAddress, and that pointer is what the kernel
// gets.  The look-up happens inside the first call on each GPU, so make that first call
// outside any stream capture.  All calls share the one array and it keeps whatever the last
// call left: the kernel overwrites every partial it later reads, so nothing needs clearing,
// but two calls that overlap on the GPU (different streams) race on it.
namespace pb {
namespace {

constexpr size_t kStaticScratchBytes = size_t(4) << 20;  // 4 MiB
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxGpus = 64;
std::mutex g_scratch_mu;
void* g_scratch_ptr[kMaxGpus] = {nullptr};

int static_scratch_for(int gpu, void** out) {
    std::lock_guard<std::mutex> lk(g_scratch_mu);
    if (!g_scratch_ptr[gpu]) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);  // `gpu` is current
        if (e != cudaSuccess || !p)
            return fail(PARAS_E_CUDA, "paras sdpa: cudaGetSymbolAddress for the static scratch failed: %s",
                        cudaGetErrorString(e));
        g_scratch_ptr[gpu] = p;
    }
    *out = g_scratch_ptr[gpu];
    return PARAS_OK;
}

}  // namespace
}  // namespace pb

extern "C" int paras_b200_sdpa_static_scratch_bytes(void) { return int(pb::kStaticScratchBytes); }

extern "C" int paras_b200_sdpa_fwd_static_scratch(const paras_sdpa_args* a) {
    pb::NvtxRange range("paras_b200_sdpa_fwd_static_scratch");
    using pb::fail;
    if (!a) return fail(PARAS_E_INVALID, "paras sdpa: null argument block");
    if (a->dtype != PARAS_F32 && a->dtype != PARAS_BF16 && a->dtype != PARAS_F16)
        return fail(PARAS_E_UNSUPPORTED, "paras sdpa: unsupported dtype %d", a->dtype);
    if (a->B < 0 || a->Hq < 0 || a->Hkv < 0 || a->Lq < 0 || a->Lk < 0 || a->D < 0)
        return fail(PARAS_E_INVALID, "paras sdpa: negative dimension");
    if (a->Hkv == 0 ? a->Hq != 0 : (a->Hq % a->Hkv) != 0)
        return fail(PARAS_E_INVALID,
                    "paras sdpa: query heads must be a multiple of key/value heads for enable_gqa");
    if (a->causal && a->mask)
        return fail(PARAS_E_INVALID, "paras sdpa: is_causal and attn_mask are mutually exclusive");
    if (a->mask && (a->mask_kind < 1 || a->mask_kind > 3))
        return fail(PARAS_E_INVALID, "paras sdpa: bad mask kind %d", a->mask_kind);
    if (pb::sdpa_wants_weights(*a))
        return fail(PARAS_E_UNSUPPORTED, "paras sdpa: dropout and the weights output go through paras_b200_sdpa_fwd");
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
        cudaGetLastError();
        return fail(PARAS_E_NODEVICE, "paras_b200: no CUDA GPU is visible; this build has no CPU fallback");
    }
    if (a->gpu < 0 || a->gpu >= count || a->gpu >= pb::kMaxGpus)
        return fail(PARAS_E_INVALID, "paras_b200: gpu ordinal %d out of range [0,%d)", a->gpu, count);
    PB_CUDA(cudaSetDevice(a->gpu));
    if (int64_t(a->B) * a->Hq * a->Lq * a->D == 0) return PARAS_OK;
    if (!a->q || !a->out || (a->Lk > 0 && (!a->k || !a->v)))
        return fail(PARAS_E_INVALID, "paras sdpa: null pointer");

    pb::Gpu g{};  // a plain descriptor: nothing is created or allocated for it
    g.ordinal = a->gpu;
    PB_CUDA(cudaDeviceGetAttribute(&g.sm_count, cudaDevAttrMultiProcessorCount, a->gpu));
    const int splits = pb::sdpa_simt_pick_splits(&g, *a);
    const int64_t rows = int64_t(a->B) * a->Hq * a->Lq;
    const size_t need = pb::split_workspace_bytes(rows, a->D, splits);
    if (need > pb::kStaticScratchBytes)
        return fail(PARAS_E_INVALID,
                    "paras sdpa: this problem needs %zu bytes of split-KV scratch but the static "
                    "scratch holds %zu; use paras_b200_sdpa_fwd with a workspace instead",
                    need, pb::kStaticScratchBytes);
    void* scratch = nullptr;
    if (need) {
        const int st = pb::static_scratch_for(a->gpu, &scratch);
        if (st != PARAS_OK) return st;
    }
    double sc = a->scale;
    if (a->flags & PARAS_SDPA_REF_SCALE) {
        float f = float(sc);
        if (a->dtype == PARAS_BF16) f = __bfloat162float(__float2bfloat16_rn(f));
        else if (a->dtype == PARAS_F16) f = __half2float(__float2half_rn(f));
        sc = f;
    }
    // a NULL stream cannot mean "the library's own stream" here (creating one would be an
    // allocation): it means the legacy default stream
    cudaStream_t s = a->stream ? static_cast<cudaStream_t>(a->stream) : cudaStreamLegacy;
    const pb::SplitWorkspace ws = pb::carve_workspace(scratch, rows, a->D, splits);
    const int st = pb::sdpa_simt_launch(&g, *a, float(sc), ws, s);
    if (st == PARAS_OK) pb::set_last_kernel(splits > 1 ? "simt_splitkv_static" : "simt");
    return st;
}


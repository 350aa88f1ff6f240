// Host runtime of libb200ew.so: device selection, caching device-memory arena,
// copies, streams/events, NVRTC kernel instantiation with a two-level cache,
// launches, the counter-based RNG state and the NCCL bridge.
//
// Only the CUDA runtime API is used (statically linked), so the library loads
// on machines without a driver; every entry point that needs a device reports
// B200_ERR_CUDA there instead of crashing.

#include "b200ew.h"

#include <cuda_runtime.h>
#include <nvrtc.h>
#include <dlfcn.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <mutex>
#include <set>
#include <string>
#include <unordered_map>
#include <vector>

namespace {

thread_local std::string g_err;

b200_status fail(b200_status code, const char *fmt, ...) {
    char buf[2048];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_err = buf;
    return code;
}

#define CU(call)                                                                     \
    do {                                                                             \
        cudaError_t e_ = (call);                                                     \
        if (e_ != cudaSuccess)                                                       \
            return fail(e_ == cudaErrorMemoryAllocation ? B200_ERR_OOM : B200_ERR_CUDA, \
                        "%s: %s", #call, cudaGetErrorString(e_));                    \
    } while (0)

// ---------------------------------------------------------------- state
struct State {
    int device = -1;
    cudaStream_t stream = nullptr;             // the library's stream of this device
    // arena
    std::multimap<uint64_t, void *> free_blocks;          // size -> ptr
    std::unordered_map<void *, uint64_t> live;            // ptr -> block size
    uint64_t in_use = 0, cached = 0, peak = 0, device_allocs = 0;
    // streams made with b200_stream_create; while there are any, a freed block waits in `parked`
    // until everything queued so far on the library's stream and on each of them has run
    std::set<cudaStream_t> user_streams;
    struct Parked { void *p; uint64_t sz; std::vector<cudaEvent_t> events; };
    std::vector<Parked> parked;
    // kernels
    std::unordered_map<std::string, std::string> headers;
    std::unordered_map<uint64_t, cudaKernel_t> kernels;   // hash(source+name+opts) -> kernel
    std::vector<cudaLibrary_t> libraries;
    uint64_t n_compiled = 0, n_disk = 0, n_mem = 0;
    // rng
    uint64_t seed = 0, launches = 0;
};
State g;
std::mutex g_mu;
std::recursive_mutex g_arena_mu;       // arena entry points may be called from any host thread (tensor finalisers)

// Parked blocks whose events have all completed (or all of them, after waiting: `wait`) go to
// the free list.  Called with the arena lock held.
void reap_parked(bool wait) {
    size_t keep = 0;
    for (size_t i = 0; i < g.parked.size(); ++i) {
        State::Parked &b = g.parked[i];
        bool done = true;
        for (cudaEvent_t e : b.events) {
            if (wait) cudaEventSynchronize(e);
            else if (cudaEventQuery(e) != cudaSuccess) { done = false; break; }
        }
        if (!done) {
            cudaGetLastError();                    // cudaErrorNotReady is not an error
            if (keep != i) g.parked[keep] = std::move(b);
            ++keep;
            continue;
        }
        for (cudaEvent_t e : b.events) cudaEventDestroy(e);
        g.free_blocks.emplace(b.sz, b.p);
        g.cached += b.sz;
    }
    g.parked.resize(keep);
}

uint64_t round_block(uint64_t bytes) {
    if (bytes == 0) bytes = 1;
    if (bytes <= (1u << 20)) return (bytes + 511) & ~uint64_t(511);
    return (bytes + (2u << 20) - 1) & ~uint64_t((2u << 20) - 1);
}

uint64_t fnv1a(const void *data, size_t n, uint64_t h = 1469598103934665603ull) {
    const unsigned char *p = static_cast<const unsigned char *>(data);
    for (size_t i = 0; i < n; ++i) { h ^= p[i]; h *= 1099511628211ull; }
    return h;
}

uint64_t splitmix64(uint64_t &x) {
    x += 0x9E3779B97F4A7C15ull;
    uint64_t z = x;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

std::string cache_dir() {
    const char *env = getenv("B200EW_CACHE_DIR");
    std::string d;
    if (env && *env) d = env;
    else {
        const char *home = getenv("HOME");
        d = std::string(home && *home ? home : "/tmp") + "/.cache/b200ew";
    }
    std::string cur;
    for (size_t i = 0; i <= d.size(); ++i) {
        if (i == d.size() || d[i] == '/') {
            if (!cur.empty()) mkdir(cur.c_str(), 0755);
        }
        if (i < d.size()) cur += d[i];
    }
    return d;
}

// ---------------------------------------------------------------- NCCL (dlopen)
struct Id128 { char bytes[128]; };
struct Nccl {
    void *lib = nullptr;
    int (*GetUniqueId)(void *) = nullptr;
    int (*CommInitRank)(void **, int, /* ncclUniqueId by value */ Id128, int) = nullptr;
    int (*CommDestroy)(void *) = nullptr;
    int (*AllReduce)(const void *, void *, size_t, int, int, void *, cudaStream_t) = nullptr;
    int (*AllGather)(const void *, void *, size_t, int, void *, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
};
Nccl nccl;

b200_status load_nccl() {
    if (nccl.lib) return B200_OK;
    const char *env = getenv("B200EW_NCCL_LIB");
    const char *names[] = {env, "libnccl.so.2", "libnccl.so"};
    for (const char *n : names) {
        if (!n || !*n) continue;
        nccl.lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (nccl.lib) break;
    }
    if (!nccl.lib) return fail(B200_ERR_NCCL, "libnccl not found (set B200EW_NCCL_LIB): %s", dlerror());
#define SYM(field, name)                                                      \
    *reinterpret_cast<void **>(&nccl.field) = dlsym(nccl.lib, name);          \
    if (!nccl.field) return fail(B200_ERR_NCCL, "symbol %s missing in libnccl", name)
    SYM(GetUniqueId, "ncclGetUniqueId");
    SYM(CommInitRank, "ncclCommInitRank");
    SYM(CommDestroy, "ncclCommDestroy");
    SYM(AllReduce, "ncclAllReduce");
    SYM(AllGather, "ncclAllGather");
    SYM(GetErrorString, "ncclGetErrorString");
#undef SYM
    return B200_OK;
}

cudaStream_t as_stream(uint64_t s) { return s ? reinterpret_cast<cudaStream_t>(s) : g.stream; }

}  // namespace

extern "C" int b200_detail_fill(void *dst, uint32_t value, int width, uint64_t count, void *stream);
extern "C" int b200_detail_reduce_full(uint64_t in, int32_t dtype, uint64_t count, int32_t op, int32_t absolute,
                                       uint64_t out, uint64_t scratch, int sm_count, void *stream);

extern "C" int b200_detail_gemm(uint64_t a, int da, int64_t a_s0, int64_t a_s1, uint64_t b, int db, int64_t b_s0,
                                int64_t b_s1, uint64_t c, int dc, int64_t c_s0, int64_t c_s1, int m, int n, int k,
                                float alpha, float beta, void *stream);

// helpers for the other translation units of the library
extern "C" void *b200_detail_stream(uint64_t stream) { return stream ? reinterpret_cast<void *>(stream) : g.stream; }
extern "C" int32_t b200_detail_fail(int32_t code, const char *message) { return fail(code, "%s", message); }

extern "C" {

int32_t b200_version(void) { return 100; }

size_t b200_last_error(char *buf, size_t n) {
    if (buf && n) {
        size_t m = g_err.size() < n - 1 ? g_err.size() : n - 1;
        memcpy(buf, g_err.data(), m);
        buf[m] = 0;
    }
    return g_err.size();
}

// ---------------------------------------------------------------- device
b200_status b200_device_count(int32_t *count) {
    if (!count) return fail(B200_ERR_INVALID, "count is null");
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) { cudaGetLastError(); n = 0; }
    *count = n;
    return B200_OK;
}

b200_status b200_init(int32_t device) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g.device == device && g.stream) return B200_OK;
    if (g.device >= 0 && g.device != device)
        return fail(B200_ERR_INVALID, "process already bound to device %d", g.device);
    CU(cudaSetDevice(device));
    CU(cudaFree(0));
    CU(cudaStreamCreateWithFlags(&g.stream, cudaStreamNonBlocking));
    g.device = device;
    return B200_OK;
}

b200_status b200_shutdown(void) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g.device < 0) return B200_OK;
    cudaDeviceSynchronize();
    {
        std::lock_guard<std::recursive_mutex> lock(g_arena_mu);
        reap_parked(true);
        g.user_streams.clear();
    }
    for (auto &kv : g.free_blocks) cudaFree(kv.second);
    for (auto &kv : g.live) cudaFree(kv.first);
    g.free_blocks.clear(); g.live.clear();
    g.in_use = g.cached = 0;
    for (auto lib : g.libraries) cudaLibraryUnload(lib);
    g.libraries.clear(); g.kernels.clear();
    if (g.stream) cudaStreamDestroy(g.stream);
    g.stream = nullptr; g.device = -1;
    return B200_OK;
}

b200_status b200_device_props_get(int32_t device, b200_device_props *out) {
    if (!out) return fail(B200_ERR_INVALID, "out is null");
    cudaDeviceProp p;
    CU(cudaGetDeviceProperties(&p, device));
    memset(out, 0, sizeof *out);
    out->sm_count = p.multiProcessorCount;
    out->cc_major = p.major; out->cc_minor = p.minor;
    out->max_smem_per_block = (int32_t)p.sharedMemPerBlockOptin;
    out->max_threads_per_sm = p.maxThreadsPerMultiProcessor;
    out->l2_bytes = p.l2CacheSize;
    int khz = 0;
    cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, device);
    out->clock_khz = khz;
    out->total_mem = p.totalGlobalMem;
    strncpy(out->name, p.name, sizeof(out->name) - 1);
    return B200_OK;
}

b200_status b200_mem_info(uint64_t *free_bytes, uint64_t *total_bytes) {
    size_t f = 0, t = 0;
    CU(cudaMemGetInfo(&f, &t));
    if (free_bytes) *free_bytes = f;
    if (total_bytes) *total_bytes = t;
    return B200_OK;
}

// ---------------------------------------------------------------- arena
b200_status b200_malloc(uint64_t bytes, uint64_t *dptr) {
    if (!dptr) return fail(B200_ERR_INVALID, "dptr is null");
    if (g.device < 0) return fail(B200_ERR_INVALID, "b200_init has not been called");
    std::lock_guard<std::recursive_mutex> lock(g_arena_mu);
    if (!g.parked.empty()) reap_parked(false);
    uint64_t sz = round_block(bytes);
    auto it = g.free_blocks.lower_bound(sz);
    void *p = nullptr;
    // reuse a cached block unless it would waste more than half of itself
    if (it != g.free_blocks.end() && it->first <= sz + sz / 2 + 4096) {
        p = it->second; sz = it->first;
        g.free_blocks.erase(it);
        g.cached -= sz;
    } else {
        cudaError_t e = cudaMalloc(&p, sz);
        if (e == cudaErrorMemoryAllocation) {        // give cached blocks back, retry once
            cudaGetLastError();
            b200_mem_trim();
            e = cudaMalloc(&p, sz);
        }
        if (e != cudaSuccess) {
            cudaGetLastError();
            return fail(e == cudaErrorMemoryAllocation ? B200_ERR_OOM : B200_ERR_CUDA,
                        "cudaMalloc(%llu): %s", (unsigned long long)sz, cudaGetErrorString(e));
        }
        g.device_allocs++;
    }
    g.live[p] = sz;
    g.in_use += sz;
    if (g.in_use > g.peak) g.peak = g.in_use;
    *dptr = reinterpret_cast<uint64_t>(p);
    return B200_OK;
}

b200_status b200_free(uint64_t dptr) {
    if (!dptr) return B200_OK;
    std::lock_guard<std::recursive_mutex> lock(g_arena_mu);
    void *p = reinterpret_cast<void *>(dptr);
    auto it = g.live.find(p);
    if (it == g.live.end()) return fail(B200_ERR_INVALID, "b200_free: %p is not a live block", p);
    uint64_t sz = it->second;
    g.live.erase(it);
    g.in_use -= sz;
    if (!g.user_streams.empty()) {
        // work on another stream may still use the block: hand it out again only after everything
        // queued so far on every stream has run (with the library's stream alone, reuse is ordered
        // by that stream and the block is free at once)
        State::Parked b;
        b.p = p; b.sz = sz;
        std::vector<cudaStream_t> streams(g.user_streams.begin(), g.user_streams.end());
        streams.push_back(g.stream);
        bool ok = true;
        for (cudaStream_t st : streams) {
            cudaEvent_t e;
            if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) { ok = false; break; }
            b.events.push_back(e);
            if (cudaEventRecord(e, st) != cudaSuccess) { ok = false; break; }
        }
        if (ok) {
            g.parked.push_back(std::move(b));
            return B200_OK;
        }
        cudaGetLastError();                        // could not mark the streams: wait for the device instead
        for (cudaEvent_t e : b.events) cudaEventDestroy(e);
        cudaDeviceSynchronize();
    }
    g.free_blocks.emplace(sz, p);
    g.cached += sz;
    return B200_OK;
}

b200_status b200_mem_trim(void) {
    std::lock_guard<std::recursive_mutex> lock(g_arena_mu);
    if (!g.parked.empty()) reap_parked(true);
    if (g.free_blocks.empty()) return B200_OK;
    cudaDeviceSynchronize();
    for (auto &kv : g.free_blocks) cudaFree(kv.second);
    g.free_blocks.clear();
    g.cached = 0;
    return B200_OK;
}

b200_status b200_mem_stats(uint64_t *in_use, uint64_t *cached, uint64_t *peak, uint64_t *allocs) {
    std::lock_guard<std::recursive_mutex> lock(g_arena_mu);
    if (in_use) *in_use = g.in_use;
    if (cached) *cached = g.cached;
    if (peak) *peak = g.peak;
    if (allocs) *allocs = g.device_allocs;
    return B200_OK;
}

b200_status b200_host_alloc(uint64_t bytes, void **hptr) {
    if (!hptr) return fail(B200_ERR_INVALID, "hptr is null");
    CU(cudaMallocHost(hptr, bytes ? bytes : 1));
    return B200_OK;
}

b200_status b200_host_free(void *hptr) {
    if (hptr) CU(cudaFreeHost(hptr));
    return B200_OK;
}

// ---------------------------------------------------------------- copies
b200_status b200_memcpy_h2d(uint64_t dst, const void *src, uint64_t bytes, uint64_t stream, int32_t sync) {
    if (!bytes) return B200_OK;
    cudaStream_t s = as_stream(stream);
    CU(cudaMemcpyAsync(reinterpret_cast<void *>(dst), src, bytes, cudaMemcpyHostToDevice, s));
    if (sync) CU(cudaStreamSynchronize(s));
    return B200_OK;
}

b200_status b200_memcpy_d2h(void *dst, uint64_t src, uint64_t bytes, uint64_t stream, int32_t sync) {
    if (!bytes) return B200_OK;
    cudaStream_t s = as_stream(stream);
    CU(cudaMemcpyAsync(dst, reinterpret_cast<const void *>(src), bytes, cudaMemcpyDeviceToHost, s));
    if (sync) CU(cudaStreamSynchronize(s));
    return B200_OK;
}

b200_status b200_memcpy_d2d(uint64_t dst, uint64_t src, uint64_t bytes, uint64_t stream) {
    if (!bytes) return B200_OK;
    CU(cudaMemcpyAsync(reinterpret_cast<void *>(dst), reinterpret_cast<const void *>(src), bytes,
                       cudaMemcpyDeviceToDevice, as_stream(stream)));
    return B200_OK;
}

b200_status b200_memset(uint64_t dst, uint32_t value, int32_t width, uint64_t count, uint64_t stream) {
    if (!count) return B200_OK;
    void *p = reinterpret_cast<void *>(dst);
    cudaStream_t s = as_stream(stream);
    if (width == 1) { CU(cudaMemsetAsync(p, (int)(value & 0xff), count, s)); return B200_OK; }
    if (width == 2 || width == 4) {
        if (dst & (uint64_t)(width - 1)) return fail(B200_ERR_INVALID, "%d-byte fill needs an aligned pointer", width);
        uint32_t b = value & 0xff;
        uint32_t rep = width == 2 ? (b | b << 8) : (b | b << 8 | b << 16 | b << 24);
        uint32_t v = width == 2 ? (value & 0xffff) : value;
        if (v == rep) { CU(cudaMemsetAsync(p, (int)b, count * width, s)); return B200_OK; }
        int e = b200_detail_fill(p, v, width, count, s);
        if (e) return fail(B200_ERR_CUDA, "fill kernel: %s", cudaGetErrorString((cudaError_t)e));
        return B200_OK;
    }
    return fail(B200_ERR_INVALID, "fill width must be 1, 2 or 4");
}

// ---------------------------------------------------------------- streams / events
b200_status b200_stream_create(uint64_t *stream) {
    if (!stream) return fail(B200_ERR_INVALID, "stream is null");
    cudaStream_t s;
    CU(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    {
        std::lock_guard<std::recursive_mutex> lock(g_arena_mu);
        g.user_streams.insert(s);
    }
    *stream = reinterpret_cast<uint64_t>(s);
    return B200_OK;
}
b200_status b200_stream_destroy(uint64_t stream) {
    if (!stream) return B200_OK;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    {
        // blocks parked with an event on this stream: let them finish before the stream goes
        std::lock_guard<std::recursive_mutex> lock(g_arena_mu);
        if (!g.parked.empty()) reap_parked(true);
        g.user_streams.erase(s);
    }
    CU(cudaStreamDestroy(s));
    return B200_OK;
}
b200_status b200_stream_sync(uint64_t stream) { CU(cudaStreamSynchronize(as_stream(stream))); return B200_OK; }
b200_status b200_stream_wait_event(uint64_t stream, uint64_t event) {
    CU(cudaStreamWaitEvent(as_stream(stream), reinterpret_cast<cudaEvent_t>(event), 0));
    return B200_OK;
}
b200_status b200_default_stream(uint64_t *stream) {
    if (!stream) return fail(B200_ERR_INVALID, "stream is null");
    *stream = reinterpret_cast<uint64_t>(g.stream);
    return B200_OK;
}
b200_status b200_event_create(uint64_t *event) {
    if (!event) return fail(B200_ERR_INVALID, "event is null");
    cudaEvent_t e;
    CU(cudaEventCreate(&e));
    *event = reinterpret_cast<uint64_t>(e);
    return B200_OK;
}
b200_status b200_event_destroy(uint64_t event) {
    if (event) CU(cudaEventDestroy(reinterpret_cast<cudaEvent_t>(event)));
    return B200_OK;
}
b200_status b200_event_record(uint64_t event, uint64_t stream) {
    CU(cudaEventRecord(reinterpret_cast<cudaEvent_t>(event), as_stream(stream)));
    return B200_OK;
}
b200_status b200_event_sync(uint64_t event) {
    CU(cudaEventSynchronize(reinterpret_cast<cudaEvent_t>(event)));
    return B200_OK;
}
b200_status b200_event_elapsed_ms(uint64_t start, uint64_t end, float *ms) {
    if (!ms) return fail(B200_ERR_INVALID, "ms is null");
    CU(cudaEventElapsedTime(ms, reinterpret_cast<cudaEvent_t>(start), reinterpret_cast<cudaEvent_t>(end)));
    return B200_OK;
}

// ---------------------------------------------------------------- kernels
b200_status b200_register_header(const char *name, const char *source) {
    if (!name || !source) return fail(B200_ERR_INVALID, "null header");
    std::lock_guard<std::mutex> lk(g_mu);
    g.headers[name] = source;
    return B200_OK;
}

static uint64_t source_hash(const char *source, const char *const *options, int32_t n_options,
                            const char *extra) {
    uint64_t h = fnv1a(source, strlen(source));
    for (int i = 0; i < n_options; ++i) h = fnv1a(options[i], strlen(options[i]) + 1, h);
    // headers take part in the key: editing a template invalidates its instances
    std::map<std::string, const std::string *> ordered;
    for (auto &kv : g.headers) ordered[kv.first] = &kv.second;
    for (auto &kv : ordered) { h = fnv1a(kv.first.data(), kv.first.size(), h); h = fnv1a(kv.second->data(), kv.second->size(), h); }
    int maj = 0, min = 0;
    nvrtcVersion(&maj, &min);
    h = fnv1a(&maj, sizeof maj, h); h = fnv1a(&min, sizeof min, h);
    if (extra) h = fnv1a(extra, strlen(extra), h);
    return h;
}

static b200_status compile_image(const char *source, const char *const *options, int32_t n_options,
                                 std::string &image, bool &from_cache) {
    uint64_t h = source_hash(source, options, n_options, "cubin");
    char fname[64];
    snprintf(fname, sizeof fname, "/%016llx.cubin", (unsigned long long)h);
    std::string path = cache_dir() + fname;
    {
        std::ifstream f(path, std::ios::binary);
        if (f) {
            image.assign(std::istreambuf_iterator<char>(f), std::istreambuf_iterator<char>());
            if (!image.empty()) { from_cache = true; g.n_disk++; return B200_OK; }
        }
    }
    from_cache = false;
    std::vector<const char *> hsrc, hname;
    for (auto &kv : g.headers) { hname.push_back(kv.first.c_str()); hsrc.push_back(kv.second.c_str()); }
    nvrtcProgram prog;
    nvrtcResult r = nvrtcCreateProgram(&prog, source, "optree_kernel.cu", (int)hsrc.size(), hsrc.data(), hname.data());
    if (r != NVRTC_SUCCESS) return fail(B200_ERR_COMPILE, "nvrtcCreateProgram: %s", nvrtcGetErrorString(r));
    std::vector<const char *> opts = {"--gpu-architecture=sm_100a", "--std=c++17", "-default-device", "-lineinfo"};
    for (int i = 0; i < n_options; ++i) opts.push_back(options[i]);
    r = nvrtcCompileProgram(prog, (int)opts.size(), opts.data());
    if (r != NVRTC_SUCCESS) {
        size_t n = 0;
        nvrtcGetProgramLogSize(prog, &n);
        std::string log(n, 0);
        nvrtcGetProgramLog(prog, &log[0]);
        nvrtcDestroyProgram(&prog);
        if (log.size() > 1800) log.resize(1800);
        return fail(B200_ERR_COMPILE, "NVRTC: %s\n%s", nvrtcGetErrorString(r), log.c_str());
    }
    size_t n = 0;
    r = nvrtcGetCUBINSize(prog, &n);
    if (r != NVRTC_SUCCESS || !n) { nvrtcDestroyProgram(&prog); return fail(B200_ERR_COMPILE, "nvrtcGetCUBINSize failed"); }
    image.resize(n);
    nvrtcGetCUBIN(prog, &image[0]);
    nvrtcDestroyProgram(&prog);
    g.n_compiled++;
    // publish atomically: write to a temp name, then rename
    std::string tmp = path + "." + std::to_string((long)getpid());
    {
        std::ofstream f(tmp, std::ios::binary);
        if (f) f.write(image.data(), (std::streamsize)image.size());
    }
    rename(tmp.c_str(), path.c_str());
    return B200_OK;
}

b200_status b200_nvrtc_compile(const char *source, const char *const *options, int32_t n_options,
                               void **image, uint64_t *image_size, int32_t *from_cache) {
    if (!source || !image || !image_size) return fail(B200_ERR_INVALID, "null argument");
    std::string img;
    bool cached = false;
    b200_status st = compile_image(source, options, n_options, img, cached);
    if (st) return st;
    void *p = malloc(img.size());
    if (!p) return fail(B200_ERR_OOM, "host malloc failed");
    memcpy(p, img.data(), img.size());
    *image = p; *image_size = img.size();
    if (from_cache) *from_cache = cached ? 1 : 0;
    return B200_OK;
}

b200_status b200_buffer_free(void *image) { free(image); return B200_OK; }

b200_status b200_kernel_get(const char *source, const char *kernel_name,
                            const char *const *options, int32_t n_options, uint64_t *kernel) {
    if (!source || !kernel_name || !kernel) return fail(B200_ERR_INVALID, "null argument");
    if (g.device < 0) return fail(B200_ERR_INVALID, "b200_init has not been called");
    uint64_t h = source_hash(source, options, n_options, kernel_name);
    auto it = g.kernels.find(h);
    if (it != g.kernels.end()) { g.n_mem++; *kernel = reinterpret_cast<uint64_t>(it->second); return B200_OK; }
    std::string img;
    bool cached = false;
    b200_status st = compile_image(source, options, n_options, img, cached);
    if (st) return st;
    cudaLibrary_t lib;
    CU(cudaLibraryLoadData(&lib, img.data(), nullptr, nullptr, 0, nullptr, nullptr, 0));
    cudaKernel_t k;
    cudaError_t e = cudaLibraryGetKernel(&k, lib, kernel_name);
    if (e != cudaSuccess) {
        cudaLibraryUnload(lib);
        return fail(B200_ERR_CUDA, "kernel %s not in module: %s", kernel_name, cudaGetErrorString(e));
    }
    g.libraries.push_back(lib);
    g.kernels[h] = k;
    *kernel = reinterpret_cast<uint64_t>(k);
    return B200_OK;
}

b200_status b200_kernel_max_smem(uint64_t kernel, int32_t bytes) {
    CU(cudaFuncSetAttribute(reinterpret_cast<const void *>(kernel),
                            cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    return B200_OK;
}

b200_status b200_kernel_occupancy(uint64_t kernel, int32_t block_threads, int32_t smem_bytes, int32_t *blocks) {
    if (!blocks) return fail(B200_ERR_INVALID, "null argument");
    int n = 0;
    CU(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, reinterpret_cast<const void *>(kernel),
                                                     block_threads, (size_t)smem_bytes));
    *blocks = n;
    return B200_OK;
}

b200_status b200_kernel_max_clusters(uint64_t kernel, int32_t block_threads, int32_t smem_bytes,
                                     int32_t cluster_size, int32_t grid_blocks, int32_t *clusters) {
    if (!clusters) return fail(B200_ERR_INVALID, "null argument");
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3((unsigned)grid_blocks, 1, 1);
    cfg.blockDim = dim3((unsigned)block_threads, 1, 1);
    cfg.dynamicSmemBytes = (size_t)smem_bytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = (unsigned)cluster_size; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr; cfg.numAttrs = 1;
    int n = 0;
    CU(cudaOccupancyMaxActiveClusters(&n, reinterpret_cast<const void *>(kernel), &cfg));
    *clusters = n;
    return B200_OK;
}

b200_status b200_cache_stats(uint64_t *compiled, uint64_t *disk_hits, uint64_t *memory_hits) {
    if (compiled) *compiled = g.n_compiled;
    if (disk_hits) *disk_hits = g.n_disk;
    if (memory_hits) *memory_hits = g.n_mem;
    return B200_OK;
}

b200_status b200_launch(uint64_t kernel, uint32_t gx, uint32_t gy, uint32_t gz,
                        uint32_t bx, uint32_t by, uint32_t bz, uint32_t smem, uint64_t stream,
                        const void *params, uint32_t params_size, uint32_t cluster_x, int32_t cooperative) {
    if (!kernel || !params) return fail(B200_ERR_INVALID, "null kernel or params");
    if (params_size > 4096) return fail(B200_ERR_INVALID, "parameter block of %u bytes exceeds 4096", params_size);
    if (!gx || !gy || !gz || !bx || !by || !bz) return fail(B200_ERR_INVALID, "empty grid or block");
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3(gx, gy, gz);
    cfg.blockDim = dim3(bx, by, bz);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = as_stream(stream);
    cudaLaunchAttribute attrs[3];
    int na = 0;
    if (cluster_x > 1) {
        attrs[na].id = cudaLaunchAttributeClusterDimension;
        attrs[na].val.clusterDim.x = cluster_x; attrs[na].val.clusterDim.y = 1; attrs[na].val.clusterDim.z = 1;
        ++na;
    }
    if (cooperative & 1) {
        attrs[na].id = cudaLaunchAttributeCooperative;
        attrs[na].val.cooperative = 1;
        ++na;
    }
    if (cooperative & 2) {
        // the kernel executes griddepcontrol.wait before it touches memory: its blocks may be
        // scheduled while the previous kernel of the stream drains
        attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = na ? attrs : nullptr;
    cfg.numAttrs = na;
    void *args[1] = {const_cast<void *>(params)};
    CU(cudaLaunchKernelExC(&cfg, reinterpret_cast<const void *>(kernel), args));
    return B200_OK;
}

// ---------------------------------------------------------------- graphs
b200_status b200_graph_begin(uint64_t stream) {
    if (g.device < 0) return fail(B200_ERR_INVALID, "b200_init has not been called");
    CU(cudaStreamBeginCapture(as_stream(stream), cudaStreamCaptureModeRelaxed));
    return B200_OK;
}

b200_status b200_graph_end(uint64_t stream, uint64_t *graph_exec) {
    if (!graph_exec) return fail(B200_ERR_INVALID, "graph_exec is null");
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(as_stream(stream), &graph);
    if (e != cudaSuccess || !graph) {
        cudaGetLastError();
        return fail(B200_ERR_CUDA, "cudaStreamEndCapture: %s", cudaGetErrorString(e));
    }
    cudaGraphExec_t exec = nullptr;
    e = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) { cudaGetLastError(); return fail(B200_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(e)); }
    *graph_exec = reinterpret_cast<uint64_t>(exec);
    return B200_OK;
}

b200_status b200_graph_launch(uint64_t graph_exec, uint64_t stream) {
    if (!graph_exec) return fail(B200_ERR_INVALID, "null graph");
    CU(cudaGraphLaunch(reinterpret_cast<cudaGraphExec_t>(graph_exec), as_stream(stream)));
    return B200_OK;
}

b200_status b200_graph_destroy(uint64_t graph_exec) {
    if (graph_exec) CU(cudaGraphExecDestroy(reinterpret_cast<cudaGraphExec_t>(graph_exec)));
    return B200_OK;
}

// ---------------------------------------------------------------- rng
b200_status b200_rng_seed(uint64_t seed) { g.seed = seed; g.launches = 0; return B200_OK; }

b200_status b200_rng_next_key(uint32_t key[2]) {
    if (!key) return fail(B200_ERR_INVALID, "key is null");
    uint64_t x = g.seed ^ 0x6A09E667F3BCC909ull;
    uint64_t a = splitmix64(x);
    uint64_t y = a ^ (g.launches * 0xD1342543DE82EF95ull);
    uint64_t b = splitmix64(y);
    key[0] = (uint32_t)(b & 0xffffffffu);
    key[1] = (uint32_t)(b >> 32);
    g.launches++;
    return B200_OK;
}

b200_status b200_rng_get_state(uint64_t state[2]) {
    if (!state) return fail(B200_ERR_INVALID, "state is null");
    state[0] = g.seed; state[1] = g.launches;
    return B200_OK;
}

b200_status b200_rng_set_state(const uint64_t state[2]) {
    if (!state) return fail(B200_ERR_INVALID, "state is null");
    g.seed = state[0]; g.launches = state[1];
    return B200_OK;
}

// ---------------------------------------------------------------- fixed-function reduction
b200_status b200_reduce_full(uint64_t in, int32_t dtype, uint64_t count, int32_t op, int32_t absolute,
                             uint64_t out, uint64_t scratch, uint64_t stream) {
    if (g.device < 0) return fail(B200_ERR_INVALID, "b200_init has not been called");
    if (!in || !out || !scratch) return fail(B200_ERR_INVALID, "null device pointer");
    if (!count) return fail(B200_ERR_INVALID, "empty input");
    if (count > 0x7fffffffull * 4) return fail(B200_ERR_INVALID, "more than 2^33 elements");
    if (dtype != B200_F32 && dtype != B200_F16 && dtype != B200_BF16)
        return fail(B200_ERR_UNSUPPORTED, "dtype %d: only f32, f16 and bf16 inputs", dtype);
    if (op != B200_SUM && op != B200_MAX && op != B200_MIN) return fail(B200_ERR_INVALID, "bad reduction op %d", op);
    if (scratch % 16) return fail(B200_ERR_INVALID, "scratch must be 16-byte aligned");
    static int sms = 0;
    if (!sms) CU(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, g.device));
    int e = b200_detail_reduce_full(in, dtype, count, op, absolute, out, scratch, sms, as_stream(stream));
    if (e) return fail(B200_ERR_CUDA, "reduce kernel: %s", cudaGetErrorString((cudaError_t)e));
    return B200_OK;
}

// ---------------------------------------------------------------- small GEMM
b200_status b200_gemm(uint64_t a, int32_t a_dtype, int64_t a_stride0, int64_t a_stride1,
                      uint64_t b, int32_t b_dtype, int64_t b_stride0, int64_t b_stride1,
                      uint64_t c, int32_t c_dtype, int64_t c_stride0, int64_t c_stride1,
                      int32_t m, int32_t n, int32_t k, float alpha, float beta, uint64_t stream) {
    if (g.device < 0) return fail(B200_ERR_INVALID, "b200_init has not been called");
    if (!a || !b || !c) return fail(B200_ERR_INVALID, "null device pointer");
    if (m <= 0 || n <= 0 || k <= 0) return fail(B200_ERR_INVALID, "empty matrix");
    for (int dt : {a_dtype, b_dtype, c_dtype})
        if (dt != B200_F32 && dt != B200_F16) return fail(B200_ERR_UNSUPPORTED, "gemm operands must be f32 or f16");
    if ((m + 15) / 16 > 65535) return fail(B200_ERR_UNSUPPORTED, "more than 1048560 rows");
    int e = b200_detail_gemm(a, a_dtype, a_stride0, a_stride1, b, b_dtype, b_stride0, b_stride1,
                             c, c_dtype, c_stride0, c_stride1, m, n, k, alpha, beta, as_stream(stream));
    if (e) return fail(B200_ERR_CUDA, "gemm kernel: %s", cudaGetErrorString((cudaError_t)e));
    return B200_OK;
}

// ---------------------------------------------------------------- NCCL bridge
b200_status b200_comm_unique_id(uint8_t id[128]) {
    b200_status st = load_nccl();
    if (st) return st;
    int r = nccl.GetUniqueId(id);
    if (r) return fail(B200_ERR_NCCL, "ncclGetUniqueId: %s", nccl.GetErrorString(r));
    return B200_OK;
}

b200_status b200_comm_init(const uint8_t id[128], int32_t n_ranks, int32_t rank, uint64_t *comm) {
    if (!comm) return fail(B200_ERR_INVALID, "comm is null");
    if (g.device < 0) return fail(B200_ERR_INVALID, "b200_init has not been called");
    b200_status st = load_nccl();
    if (st) return st;
    Id128 uid;
    memcpy(uid.bytes, id, 128);
    void *c = nullptr;
    int r = nccl.CommInitRank(&c, n_ranks, uid, rank);
    if (r) return fail(B200_ERR_NCCL, "ncclCommInitRank: %s", nccl.GetErrorString(r));
    *comm = reinterpret_cast<uint64_t>(c);
    return B200_OK;
}

b200_status b200_comm_destroy(uint64_t comm) {
    if (!comm) return B200_OK;
    int r = nccl.CommDestroy(reinterpret_cast<void *>(comm));
    if (r) return fail(B200_ERR_NCCL, "ncclCommDestroy: %s", nccl.GetErrorString(r));
    return B200_OK;
}

static int nccl_dtype(int32_t dt) {   // ncclDataType_t values
    switch (dt) {
        case B200_F32: return 7;  case B200_F16: return 6;  case B200_BF16: return 9;
        case B200_I32: return 2;  case B200_U32: return 3;  case B200_I8: return 0; case B200_U8: return 1;
        default: return -1;
    }
}

b200_status b200_allreduce(uint64_t comm, uint64_t send, uint64_t recv, uint64_t count,
                           int32_t dtype, int32_t op, uint64_t stream) {
    if (!comm) return fail(B200_ERR_INVALID, "null communicator");
    int dt = nccl_dtype(dtype);
    if (dt < 0) return fail(B200_ERR_UNSUPPORTED, "dtype %d has no NCCL type", dtype);
    int rop = op == B200_SUM ? 0 : op == B200_MAX ? 2 : op == B200_MIN ? 3 : -1;   // ncclSum/Max/Min
    if (rop < 0) return fail(B200_ERR_INVALID, "bad reduction op %d", op);
    int r = nccl.AllReduce(reinterpret_cast<const void *>(send), reinterpret_cast<void *>(recv), count, dt, rop,
                           reinterpret_cast<void *>(comm), as_stream(stream));
    if (r) return fail(B200_ERR_NCCL, "ncclAllReduce: %s", nccl.GetErrorString(r));
    return B200_OK;
}

b200_status b200_allgather(uint64_t comm, uint64_t send, uint64_t recv, uint64_t send_bytes, uint64_t stream) {
    if (!comm) return fail(B200_ERR_INVALID, "null communicator");
    int r = nccl.AllGather(reinterpret_cast<const void *>(send), reinterpret_cast<void *>(recv), send_bytes, 0 /* ncclInt8 */,
                           reinterpret_cast<void *>(comm), as_stream(stream));
    if (r) return fail(B200_ERR_NCCL, "ncclAllGather: %s", nccl.GetErrorString(r));
    return B200_OK;
}

// ---------------------------------------------------------------- exchange areas (peer memory)
struct Xchg {
    void *local = nullptr;
    void *table = nullptr;
    std::vector<void *> opened;
};
static std::unordered_map<uint64_t, Xchg> g_xchg;

b200_status b200_xchg_create(uint64_t comm, int32_t n_ranks, int32_t rank, uint64_t bytes,
                             uint64_t *local, uint64_t *table) {
    if (!comm || n_ranks < 1 || rank < 0 || rank >= n_ranks || !local || !table || !bytes)
        return fail(B200_ERR_INVALID, "b200_xchg_create: bad arguments");
    if (g.device < 0) return fail(B200_ERR_INVALID, "b200_init has not been called");
    Xchg x;
    CU(cudaMalloc(&x.local, bytes));
    CU(cudaMemset(x.local, 0, bytes));
    CU(cudaDeviceSynchronize());
    cudaIpcMemHandle_t mine;
    CU(cudaIpcGetMemHandle(&mine, x.local));
    // the handles travel over the communicator: staged in device memory, gathered, read back
    const size_t hb = sizeof(cudaIpcMemHandle_t);
    void *stage = nullptr;
    CU(cudaMalloc(&stage, hb * (size_t)(n_ranks + 1)));
    CU(cudaMemcpy(stage, &mine, hb, cudaMemcpyHostToDevice));
    b200_status st = b200_allgather(comm, reinterpret_cast<uint64_t>(stage),
                                    reinterpret_cast<uint64_t>(static_cast<char *>(stage) + hb), hb,
                                    reinterpret_cast<uint64_t>(g.stream));
    if (st != B200_OK) { cudaFree(stage); cudaFree(x.local); return st; }
    CU(cudaStreamSynchronize(g.stream));
    std::vector<cudaIpcMemHandle_t> all(n_ranks);
    CU(cudaMemcpy(all.data(), static_cast<char *>(stage) + hb, hb * (size_t)n_ranks, cudaMemcpyDeviceToHost));
    CU(cudaFree(stage));
    std::vector<uint64_t> bases(n_ranks);
    for (int r = 0; r < n_ranks; ++r) {
        if (r == rank) { bases[r] = reinterpret_cast<uint64_t>(x.local); continue; }
        void *p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, all[r], cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            cudaGetLastError();
            for (void *q : x.opened) cudaIpcCloseMemHandle(q);
            cudaFree(x.local);
            return fail(B200_ERR_CUDA, "cudaIpcOpenMemHandle(rank %d): %s", r, cudaGetErrorString(e));
        }
        x.opened.push_back(p);
        bases[r] = reinterpret_cast<uint64_t>(p);
    }
    CU(cudaMalloc(&x.table, sizeof(uint64_t) * (size_t)n_ranks));
    CU(cudaMemcpy(x.table, bases.data(), sizeof(uint64_t) * (size_t)n_ranks, cudaMemcpyHostToDevice));
    *local = reinterpret_cast<uint64_t>(x.local);
    *table = reinterpret_cast<uint64_t>(x.table);
    std::lock_guard<std::mutex> lock(g_mu);
    g_xchg[*local] = x;
    return B200_OK;
}

b200_status b200_xchg_destroy(uint64_t local) {
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_xchg.find(local);
    if (it == g_xchg.end()) return fail(B200_ERR_INVALID, "b200_xchg_destroy: unknown exchange area");
    cudaDeviceSynchronize();
    for (void *q : it->second.opened) cudaIpcCloseMemHandle(q);
    cudaFree(it->second.table);
    cudaFree(it->second.local);
    g_xchg.erase(it);
    return B200_OK;
}

}  // extern "C"

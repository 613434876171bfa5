// Runtime of the backend: per-device stream pool, stream-ordered pool allocator, host<->device
// copies, error text. Replaces the reference's src/cuda/mem.cu and src/cuda/streams.cu.
#include "common.cuh"

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

namespace tnb {

std::atomic<uint64_t> g_launches{0};

char* error_buffer() {
    static thread_local char buffer[512] = {0};
    return buffer;
}

tn_status fail(tn_status code, const char* fmt, ...) {
    va_list args;
    va_start(args, fmt);
    vsnprintf(error_buffer(), 512, fmt, args);
    va_end(args);
    return code;
}

int env_knob(const char* name, int fallback) {
    struct Entry { const char* name; int value; bool set; };
    static std::mutex mutex;
    static std::vector<Entry> seen;
    std::lock_guard<std::mutex> lock(mutex);
    for (const Entry& e : seen)
        if (e.name == name) return e.set ? e.value : fallback;
    const char* v = getenv(name);
    const int n = (v && *v) ? atoi(v) : 0;
    seen.push_back({name, n, n > 0});
    return n > 0 ? n : fallback;
}

tn_status after_launch(const char* what) {
    count_launch();
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return fail(TN_ERROR, "launch of %s failed: %s", what, cudaGetErrorString(err));
    return TN_SUCCESS;
}

// ------------------------------------------------------------------ devices ----------
namespace {

struct DeviceState {
    std::vector<cudaStream_t> idle;  // LIFO: the most recently returned stream is handed out next
    cudaMemPool_t pool = nullptr;    // the backend's own stream-ordered pool (created on first use)
    int sms = 0;
};

struct Runtime {
    std::mutex mutex;
    std::vector<DeviceState> devices;
    bool counted = false;
    cudaError_t count_error = cudaSuccess;

    tn_status ensure_counted() {
        if (!counted) {
            int n = 0;
            count_error = cudaGetDeviceCount(&n);
            if (count_error != cudaSuccess) {
                n = 0;
                cudaGetLastError();
            }
            devices.resize(n);
            counted = true;
        }
        return TN_SUCCESS;
    }
};

Runtime& runtime() {
    static Runtime* instance = new Runtime();  // never destroyed: streams outlive static teardown
    return *instance;
}

}  // namespace

// ---- write-combined element assignments -------------------------------------------------------
// The front-end fills a device tensor from an initializer list one element at a time
// (Tensor::assign, src/tensor.cpp:34-44: one cuda::copyFromHost of dsizeof(dtype) bytes per element).
// tn_assign_from_host gathers such writes while they extend one contiguous device range and sends
// the range as ONE copy as soon as anything else happens on this thread: every entry point of the
// library passes through use_device(), which flushes first, so program order is kept. The pending
// run belongs to the calling thread: a thread must flush (any entry point, or tn_flush_assignments)
// before it ends or hands the tensor to another thread.
namespace {
struct PendingAssign {
    int device = -1;
    char* begin = nullptr;
    std::vector<char> bytes;
};
thread_local PendingAssign t_pending;
thread_local bool t_flushing = false;
std::atomic<uint64_t> g_h2d_copies{0};
constexpr size_t kMaxPendingBytes = size_t(4) << 20;
}  // namespace

static tn_status pop_stream(int id, cudaStream_t* out);
static void put_stream(int id, cudaStream_t stream);

tn_status flush_assignments() {
    if (t_flushing || t_pending.bytes.empty()) return TN_SUCCESS;
    t_flushing = true;
    cudaStream_t s = nullptr;
    tn_status st = pop_stream(t_pending.device, &s);
    if (st == TN_SUCCESS) {
        // pageable source: the runtime stages it before the call returns, so the buffer can be reused
        const cudaError_t err = cudaMemcpyAsync(t_pending.begin, t_pending.bytes.data(), t_pending.bytes.size(), cudaMemcpyHostToDevice, s);
        g_h2d_copies.fetch_add(1, std::memory_order_relaxed);
        put_stream(t_pending.device, s);
        if (err != cudaSuccess) st = fail(TN_ERROR, "H2D copy of gathered assignments failed: %s", cudaGetErrorString(err));
    }
    t_pending.bytes.clear();
    t_pending.begin = nullptr;
    t_pending.device = -1;
    t_flushing = false;
    return st;
}

tn_status use_device(int id) {
    TN_TRY(flush_assignments());
    // Always re-issued: other libraries in the process (torch) may have changed the thread's
    // current device since the last call; cudaSetDevice on the current device is a fast path.
    Runtime& rt = runtime();
    {
        std::lock_guard<std::mutex> lock(rt.mutex);
        rt.ensure_counted();
        if (id < 0 || id >= (int)rt.devices.size())
            return fail(TN_ERROR, "device id %d out of range (%d visible)", id, (int)rt.devices.size());
    }
    TN_CUDA(cudaSetDevice(id));
    return TN_SUCCESS;
}

tn_status use_device_of(const tn_tensor_t* t) {
    if (t == nullptr) return fail(TN_ERROR, "null tensor");
    if (t->environment.kind != TN_DEVICE)
        return fail(TN_INCOMPATIBLE_DEVICES, "device entry point called with a host tensor (no CPU fallback)");
    return use_device(t->environment.resource.device.id);
}

int sm_count() {
    Runtime& rt = runtime();
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    std::lock_guard<std::mutex> lock(rt.mutex);
    rt.ensure_counted();
    if (dev >= (int)rt.devices.size()) return 148;
    DeviceState& ds = rt.devices[dev];
    if (ds.sms == 0) {
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
        ds.sms = sms;
    }
    return ds.sms;
}

// SMs that the persistent tensor-core kernels leave free (see tn_set_sm_margin).
static std::atomic<int> g_sm_margin{0};
int sm_margin() { return g_sm_margin.load(std::memory_order_relaxed); }

// The backend allocates from a memory pool of its own, so that keeping freed blocks (release
// threshold = unlimited: the allocate/free pair around every expression temporary never goes back
// to the driver) does not change the behaviour of the process-wide default pool, which other
// libraries in the process allocate from.
static tn_status device_pool(int id, cudaMemPool_t* out) {
    Runtime& rt = runtime();
    std::lock_guard<std::mutex> lock(rt.mutex);
    rt.ensure_counted();
    if (id < 0 || id >= (int)rt.devices.size()) return fail(TN_ERROR, "device id %d out of range", id);
    DeviceState& ds = rt.devices[id];
    if (!ds.pool) {
        cudaMemPoolProps props = {};
        props.allocType = cudaMemAllocationTypePinned;
        props.handleTypes = cudaMemHandleTypeNone;
        props.location.type = cudaMemLocationTypeDevice;
        props.location.id = id;
        cudaMemPool_t pool = nullptr;
        TN_CUDA(cudaMemPoolCreate(&pool, &props));
        uint64_t threshold = UINT64_MAX;
        TN_CUDA(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &threshold));
        ds.pool = pool;
    }
    *out = ds.pool;
    return TN_SUCCESS;
}

tn_status scratch_alloc(void** ptr, size_t nbytes, cudaStream_t stream) {
    int dev = 0;
    TN_CUDA(cudaGetDevice(&dev));
    cudaMemPool_t pool = nullptr;
    TN_TRY(device_pool(dev, &pool));
    TN_CUDA(cudaMallocFromPoolAsync(ptr, nbytes ? nbytes : 1, pool, stream));
    return TN_SUCCESS;
}

tn_status scratch_free(void* ptr, cudaStream_t stream) {
    TN_CUDA(cudaFreeAsync(ptr, stream));
    return TN_SUCCESS;
}

static tn_status pop_stream(int id, cudaStream_t* out) {
    TN_TRY(use_device(id));
    Runtime& rt = runtime();
    {
        std::lock_guard<std::mutex> lock(rt.mutex);
        DeviceState& ds = rt.devices[id];
        if (!ds.idle.empty()) {
            *out = ds.idle.back();
            ds.idle.pop_back();
            return TN_SUCCESS;
        }
    }
    // Blocking with respect to the legacy default stream, as the reference's pool streams are
    // (cudaStreamCreate, src/cuda/streams.cu:27-33): work a caller puts on stream 0 is ordered after
    // the copies and allocations this library queued on its pool stream.
    TN_CUDA(cudaStreamCreate(out));
    return TN_SUCCESS;
}

static void put_stream(int id, cudaStream_t stream) {
    Runtime& rt = runtime();
    std::lock_guard<std::mutex> lock(rt.mutex);
    if (id >= 0 && id < (int)rt.devices.size()) rt.devices[id].idle.push_back(stream);
}

}  // namespace tnb

using namespace tnb;

extern "C" {

size_t tn_dtype_size(tn_dtype dtype) { return (size_t)dtype_bytes((int)dtype); }

const char* tn_last_error(void) { return error_buffer(); }

tn_status tn_set_sm_margin(int sms) {
    if (sms < 0 || sms > 64) return fail(TN_ERROR, "tn_set_sm_margin: %d is not in 0..64", sms);
    g_sm_margin.store(sms, std::memory_order_relaxed);
    return TN_SUCCESS;
}

uint64_t tn_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

tn_status tn_device_count(int* count) {
    if (!count) return fail(TN_ERROR, "null count");
    Runtime& rt = runtime();
    std::lock_guard<std::mutex> lock(rt.mutex);
    rt.ensure_counted();
    *count = (int)rt.devices.size();
    if (rt.count_error != cudaSuccess)
        return fail(TN_ERROR, "cudaGetDeviceCount failed: %s", cudaGetErrorString(rt.count_error));
    return TN_SUCCESS;
}

tn_status tn_set_device(int id) { return use_device(id); }

tn_status tn_stream_pop(const tn_device_t* device, tn_stream_t* stream) {
    if (!device || !stream) return fail(TN_ERROR, "null argument");
    cudaStream_t s = nullptr;
    TN_TRY(pop_stream(device->id, &s));
    stream->address = reinterpret_cast<uintptr_t>(s);
    return TN_SUCCESS;
}

tn_status tn_stream_put(const tn_device_t* device, tn_stream_t stream) {
    if (!device) return fail(TN_ERROR, "null device");
    put_stream(device->id, as_cuda(stream));
    return TN_SUCCESS;
}

tn_status tn_stream_synchronize(tn_stream_t stream) {
    TN_TRY(flush_assignments());
    TN_CUDA(cudaStreamSynchronize(as_cuda(stream)));
    return surface_device_aborts();
}

tn_status tn_allocate(const tn_device_t* device, size_t nbytes, void** address) {
    if (!device || !address) return fail(TN_NULL_ALLOCATOR, "null argument");
    *address = nullptr;
    cudaStream_t s = nullptr;
    TN_TRY(pop_stream(device->id, &s));
    cudaMemPool_t pool = nullptr;
    tn_status st = device_pool(device->id, &pool);
    if (st == TN_SUCCESS) {
        cudaError_t err = cudaMallocFromPoolAsync(address, nbytes ? nbytes : 1, pool, s);
        if (err != cudaSuccess) {
            cudaGetLastError();
            *address = nullptr;
            st = fail(TN_ERROR, "device allocation of %zu bytes failed: %s", nbytes, cudaGetErrorString(err));
        }
    }
    put_stream(device->id, s);
    return st;
}

tn_status tn_deallocate(const tn_device_t* device, void* address) {
    if (!device) return fail(TN_NULL_ALLOCATOR, "null device");
    if (!address) return TN_SUCCESS;
    cudaStream_t s = nullptr;
    TN_TRY(pop_stream(device->id, &s));
    cudaError_t err = cudaFreeAsync(address, s);
    put_stream(device->id, s);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(TN_ERROR, "cudaFreeAsync failed: %s", cudaGetErrorString(err));
    }
    return TN_SUCCESS;
}

tn_status tn_copy_from_host(const tn_device_t* device, const void* host, void* dev, size_t nbytes) {
    if (!device) return fail(TN_ERROR, "null device");
    cudaStream_t s = nullptr;
    TN_TRY(pop_stream(device->id, &s));
    // A pageable source is staged by the CUDA runtime before the call returns, so the caller may reuse
    // `host` at once (the reference relies on the same property, src/cuda/mem.cu:38-44). A PINNED
    // source is read by the copy engine later, in stream order: it must stay unchanged until the pool
    // stream has passed the copy (tn_stream_synchronize, or any synchronising call).
    cudaError_t err = cudaMemcpyAsync(dev, host, nbytes, cudaMemcpyHostToDevice, s);
    g_h2d_copies.fetch_add(1, std::memory_order_relaxed);
    put_stream(device->id, s);
    if (err != cudaSuccess) return fail(TN_ERROR, "H2D copy failed: %s", cudaGetErrorString(err));
    return TN_SUCCESS;
}

tn_status tn_assign_from_host(const tn_device_t* device, const void* host, void* dev, size_t nbytes) {
    if (!device || !host || !dev) return fail(TN_ERROR, "null argument");
    if (nbytes == 0) return TN_SUCCESS;
    char* target = static_cast<char*>(dev);
    const bool extends = !t_pending.bytes.empty() && t_pending.device == device->id && target == t_pending.begin + t_pending.bytes.size() &&
                         t_pending.bytes.size() + nbytes <= kMaxPendingBytes;
    if (!extends) {
        TN_TRY(flush_assignments());
        t_pending.device = device->id;
        t_pending.begin = target;
    }
    const char* src = static_cast<const char*>(host);
    t_pending.bytes.insert(t_pending.bytes.end(), src, src + nbytes);
    return TN_SUCCESS;
}

tn_status tn_flush_assignments(void) { return flush_assignments(); }

uint64_t tn_h2d_copy_count(void) { return g_h2d_copies.load(std::memory_order_relaxed); }

tn_status tn_copy_to_host(const tn_device_t* device, const void* dev, void* host, size_t nbytes) {
    if (!device) return fail(TN_ERROR, "null device");
    cudaStream_t s = nullptr;
    TN_TRY(pop_stream(device->id, &s));
    cudaError_t err = cudaMemcpyAsync(host, dev, nbytes, cudaMemcpyDeviceToHost, s);
    if (err == cudaSuccess) err = cudaStreamSynchronize(s);
    put_stream(device->id, s);
    if (err != cudaSuccess) return fail(TN_ERROR, "D2H copy failed: %s", cudaGetErrorString(err));
    return surface_device_aborts();
}

tn_status tn_copy_from_host_async(const tn_device_t* device, const void* host, void* dev, size_t nbytes, tn_stream_t stream) {
    if (!device) return fail(TN_ERROR, "null device");
    TN_TRY(use_device(device->id));
    const cudaError_t err = cudaMemcpyAsync(dev, host, nbytes, cudaMemcpyHostToDevice, as_cuda(stream));
    if (err != cudaSuccess) return fail(TN_ERROR, "H2D copy failed: %s", cudaGetErrorString(err));
    return TN_SUCCESS;
}

tn_status tn_copy_to_host_async(const tn_device_t* device, const void* dev, void* host, size_t nbytes, tn_stream_t stream) {
    if (!device) return fail(TN_ERROR, "null device");
    TN_TRY(use_device(device->id));
    const cudaError_t err = cudaMemcpyAsync(host, dev, nbytes, cudaMemcpyDeviceToHost, as_cuda(stream));
    if (err != cudaSuccess) return fail(TN_ERROR, "D2H copy failed: %s", cudaGetErrorString(err));
    return TN_SUCCESS;
}

tn_status tn_compare_from_host(const tn_device_t* device, const void* host, const void* dev,
                               size_t nbytes, int* equal) {
    if (!device || !equal) return fail(TN_ERROR, "null argument");
    void* staging = malloc(nbytes ? nbytes : 1);
    if (!staging) return fail(TN_ERROR, "out of host memory");
    tn_status st = tn_copy_to_host(device, dev, staging, nbytes);
    if (st == TN_SUCCESS) *equal = memcmp(host, staging, nbytes) == 0;
    free(staging);
    return st;
}

tn_status tn_copy(const tn_tensor_t* src, tn_tensor_t* dst, size_t nbytes, tn_stream_t stream) {
    if (!src || !dst) return fail(TN_ERROR, "null tensor");
    cudaStream_t s = as_cuda(stream);
    const bool src_dev = src->environment.kind == TN_DEVICE;
    const bool dst_dev = dst->environment.kind == TN_DEVICE;
    if (src_dev) TN_TRY(use_device(src->environment.resource.device.id));
    else if (dst_dev) TN_TRY(use_device(dst->environment.resource.device.id));
    if (!src_dev && dst_dev) {
        if (src->environment.resource.host.traits & TN_PINNED)
            TN_CUDA(cudaMemcpyAsync(dst->address, src->address, nbytes, cudaMemcpyHostToDevice, s));
        else {
            TN_CUDA(cudaMemcpyAsync(dst->address, src->address, nbytes, cudaMemcpyHostToDevice, s));
            TN_CUDA(cudaStreamSynchronize(s));
        }
    } else if (src_dev && !dst_dev) {
        TN_CUDA(cudaMemcpyAsync(dst->address, src->address, nbytes, cudaMemcpyDeviceToHost, s));
        if (!(dst->environment.resource.host.traits & TN_PINNED)) TN_CUDA(cudaStreamSynchronize(s));
    } else if (src_dev && dst_dev) {
        TN_CUDA(cudaMemcpyAsync(dst->address, src->address, nbytes, cudaMemcpyDefault, s));
    } else {
        memcpy(dst->address, src->address, nbytes);
    }
    return TN_SUCCESS;
}

tn_status tn_host_allocate_pinned(size_t nbytes, void** address) {
    if (!address) return fail(TN_NULL_ALLOCATOR, "null address");
    TN_CUDA(cudaHostAlloc(address, nbytes ? nbytes : 1, cudaHostAllocDefault));
    return TN_SUCCESS;
}

tn_status tn_host_free_pinned(void* address) {
    if (!address) return TN_SUCCESS;
    TN_CUDA(cudaFreeHost(address));
    return TN_SUCCESS;
}

}  // extern "C"

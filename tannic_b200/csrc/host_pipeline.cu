// Host-to-host transfer path: a fused elementwise program whose operands and result live in HOST
// memory. The rows are cut into chunks; the host-to-device copy of chunk c + 1, the kernel of chunk c
// and the device-to-host copy of chunk c - 1 run at the same time on three private streams (PCIe is
// full duplex), so a call costs about one direction's transfer time instead of both plus the kernel.
// The reference moves a tensor with one synchronous cudaMemcpy per call (src/cuda/mem.cu:54-90), has
// no pinned host allocator (src/resources.cpp:24-38 throws "not supported yet") and no notion of the
// host memory node a GPU is attached to (include/tannic/resources.hpp:194-197 leaves `Mesh` as a TODO).
#include "common.cuh"

#include <cerrno>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include <sched.h>
#include <sys/syscall.h>
#include <unistd.h>

namespace tnb {
namespace {

constexpr int kMaxChunks = 64;

constexpr int kMaxDevices = 64;

// Streams, events and staging memory of one device; created on first use, kept until exit. Calls on
// one device are serialised by the device's own mutex, calls on different devices run side by side.
struct Pipeline {
    std::mutex mutex;
    bool ready = false;
    cudaStream_t in = nullptr, run = nullptr, out = nullptr;
    cudaEvent_t arrived[kMaxChunks] = {}, done[kMaxChunks] = {};
    void* stage_in[TN_PROGRAM_MAX_INPUTS] = {};
    size_t stage_in_bytes[TN_PROGRAM_MAX_INPUTS] = {};
    void* stage_out = nullptr;
    size_t stage_out_bytes = 0;
};

Pipeline g_pipelines[kMaxDevices];

tn_status prepare(Pipeline& p) {
    if (p.ready) return TN_SUCCESS;
    TN_CUDA(cudaStreamCreateWithFlags(&p.in, cudaStreamNonBlocking));
    TN_CUDA(cudaStreamCreateWithFlags(&p.run, cudaStreamNonBlocking));
    TN_CUDA(cudaStreamCreateWithFlags(&p.out, cudaStreamNonBlocking));
    for (int c = 0; c < kMaxChunks; ++c) {
        TN_CUDA(cudaEventCreateWithFlags(&p.arrived[c], cudaEventDisableTiming));
        TN_CUDA(cudaEventCreateWithFlags(&p.done[c], cudaEventDisableTiming));
    }
    p.ready = true;
    return TN_SUCCESS;
}

// Staging memory only grows; a call that needs no more than the last one allocates nothing.
tn_status grow(void** ptr, size_t* have, size_t want) {
    if (*have >= want) return TN_SUCCESS;
    if (*ptr) TN_CUDA(cudaFree(*ptr));
    *ptr = nullptr;
    *have = 0;
    TN_CUDA(cudaMalloc(ptr, want));
    *have = want;
    return TN_SUCCESS;
}

bool dense_row_major(const tn_tensor_t* t) {
    int64_t expect = 1;
    for (int d = t->rank - 1; d >= 0; --d) {
        if (t->shape.sizes[d] != 1 && t->strides.sizes[d] != expect) return false;
        expect *= (int64_t)t->shape.sizes[d];
    }
    return true;
}

// NUMA node the device's PCIe function hangs off, or -1 when the platform does not say.
int numa_node_of(int device) {
    char bus[32] = {0};
    if (cudaDeviceGetPCIBusId(bus, sizeof(bus), device) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    for (char* c = bus; *c; ++c)
        if (*c >= 'A' && *c <= 'Z') *c = (char)(*c - 'A' + 'a');
    char path[128];
    snprintf(path, sizeof(path), "/sys/bus/pci/devices/%s/numa_node", bus);
    FILE* f = fopen(path, "r");
    if (!f) return -1;
    int node = -1;
    if (fscanf(f, "%d", &node) != 1) node = -1;
    fclose(f);
    return node;
}

// "0-15,32-47" -> cpu set. Returns the number of CPUs found.
int parse_cpulist(const char* text, cpu_set_t* set) {
    CPU_ZERO(set);
    int found = 0;
    const char* p = text;
    while (*p) {
        char* end = nullptr;
        long a = strtol(p, &end, 10);
        if (end == p) break;
        long b = a;
        p = end;
        if (*p == '-') {
            b = strtol(p + 1, &end, 10);
            p = end;
        }
        for (long c = a; c <= b && c < CPU_SETSIZE; ++c) {
            CPU_SET((int)c, set);
            ++found;
        }
        if (*p == ',') ++p;
        else break;
    }
    return found;
}

constexpr int kMpolDefault = 0, kMpolPreferred = 1, kMpolInterleave = 3;
// node >= 0: that node; node < 0 with kMpolInterleave: every node up to `last_node`
long set_mempolicy_node(int mode, int node, int last_node = -1) {
    unsigned long mask[16] = {0};  // up to 1024 nodes
    const int bits = 8 * (int)sizeof(unsigned long);
    if (node >= 0 && node < 1024) mask[node / bits] |= 1ul << (node % bits);
    for (int n = 0; node < 0 && n <= last_node && n < 1024; ++n) mask[n / bits] |= 1ul << (n % bits);
    return syscall(SYS_set_mempolicy, mode, mode == kMpolDefault ? nullptr : mask, mode == kMpolDefault ? 0ul : 1025ul);
}

// Highest memory node the kernel reports online (0 on a single-node host, -1 when it does not say).
int last_online_node() {
    FILE* f = fopen("/sys/devices/system/node/online", "r");
    if (!f) return -1;
    char text[256] = {0};
    const bool got = fgets(text, sizeof(text), f) != nullptr;
    fclose(f);
    if (!got) return -1;
    int last = -1;
    for (const char* p = text; *p;) {
        char* end = nullptr;
        const long v = strtol(p, &end, 10);
        if (end == p) break;
        if (v > last) last = (int)v;
        p = (*end == '-' || *end == ',') ? end + 1 : end;
        if (*end != '-' && *end != ',') break;
    }
    return last;
}

}  // namespace
}  // namespace tnb

using namespace tnb;

extern "C" {

tn_status tn_device_numa_node(const tn_device_t* device, int* node) {
    if (!device || !node) return fail(TN_ERROR, "null argument");
    TN_TRY(use_device(device->id));
    *node = numa_node_of(device->id);
    return TN_SUCCESS;
}

int tn_host_memory_nodes(void) { return last_online_node() + 1; }

tn_status tn_bind_thread_near(const tn_device_t* device, int* node) {
    if (!device) return fail(TN_ERROR, "null device");
    TN_TRY(use_device(device->id));
    const int n = numa_node_of(device->id);
    if (node) *node = n;
    if (n < 0) return TN_SUCCESS;  // the platform names no node: nothing to bind to
    char path[96];
    snprintf(path, sizeof(path), "/sys/devices/system/node/node%d/cpulist", n);
    FILE* f = fopen(path, "r");
    if (!f) return TN_SUCCESS;
    char text[1024] = {0};
    const bool got = fgets(text, sizeof(text), f) != nullptr;
    fclose(f);
    cpu_set_t set;
    if (!got || parse_cpulist(text, &set) == 0) return TN_SUCCESS;
    // keep to the CPUs the process is allowed on (a container's cpuset may be narrower)
    cpu_set_t allowed;
    if (sched_getaffinity(0, sizeof(allowed), &allowed) == 0) {
        cpu_set_t both;
        CPU_AND(&both, &set, &allowed);
        if (CPU_COUNT(&both) == 0) return TN_SUCCESS;
        set = both;
    }
    if (sched_setaffinity(0, sizeof(set), &set) != 0) return fail(TN_ERROR, "sched_setaffinity failed: %s", strerror(errno));
    return TN_SUCCESS;
}

tn_status tn_host_allocate_pinned_near(const tn_device_t* device, size_t nbytes, void** address) {
    if (!device || !address) return fail(TN_NULL_ALLOCATOR, "null argument");
    TN_TRY(use_device(device->id));
    const int node = numa_node_of(device->id);
    // Pages are placed when they are first touched; cudaHostAlloc touches them while it pins them, so the
    // policy is set around the call and put back afterwards: the device's own node where the platform
    // names it; otherwise, on a host with several memory nodes, the pages are interleaved over all of
    // them, so that the GPUs of a box do not all stream through the memory controllers of whichever node
    // the ranks happened to start on. A kernel or container that refuses the policy call leaves the
    // default placement, which is what tn_host_allocate_pinned gives.
    bool placed = false;
    if (node >= 0) placed = set_mempolicy_node(kMpolPreferred, node) == 0;
    else if (const int last = last_online_node(); last > 0) placed = set_mempolicy_node(kMpolInterleave, -1, last) == 0;
    const cudaError_t err = cudaHostAlloc(address, nbytes ? nbytes : 1, cudaHostAllocDefault);
    if (placed) set_mempolicy_node(kMpolDefault, -1);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(TN_ERROR, "cudaHostAlloc(%zu) failed: %s", nbytes, cudaGetErrorString(err));
    }
    return TN_SUCCESS;
}

tn_status tn_eltwise_program_host(const tn_device_t* device, const tn_tensor_t* const* inputs, int n_inputs,
                                  const tn_eltwise_node_t* nodes, int n_nodes, tn_tensor_t* dst, int chunks) {
    if (!device || !inputs || !nodes || !dst) return fail(TN_ERROR, "null argument");
    if (n_inputs < 1 || n_inputs > TN_PROGRAM_MAX_INPUTS) return fail(TN_ERROR, "program with %d inputs is out of range", n_inputs);
    if (dst->environment.kind != TN_HOST || !dense_row_major(dst)) return fail(TN_ERROR, "the result must be a dense host tensor");
    const size_t es = (size_t)dtype_bytes(dst->dtype);
    if (es == 0) return fail(TN_UNSUPPORTED_DTYPE, "dtype %d", (int)dst->dtype);
    for (int k = 0; k < n_inputs; ++k) {
        if (!inputs[k]) return fail(TN_ERROR, "null input %d", k);
        if (inputs[k]->environment.kind != TN_HOST || !dense_row_major(inputs[k])) return fail(TN_ERROR, "input %d must be a dense host tensor", k);
        if (inputs[k]->dtype != dst->dtype) return fail(TN_UNSUPPORTED_DTYPE, "input %d has dtype %d, result has %d", k, (int)inputs[k]->dtype, (int)dst->dtype);
    }
    if (dst->size == 0) return TN_SUCCESS;
    TN_TRY(use_device(device->id));
    if (device->id >= kMaxDevices) return fail(TN_ERROR, "device id %d is beyond the %d devices the host pipeline keeps state for", device->id, kMaxDevices);
    Pipeline& p = g_pipelines[device->id];
    std::lock_guard<std::mutex> lock(p.mutex);
    TN_TRY(prepare(p));

    // an input is cut along its rows when it has the result's rank and leading extent; anything smaller
    // (a broadcast row, a scalar) goes over whole before the first chunk
    const int64_t rows = dst->rank >= 2 ? (int64_t)dst->shape.sizes[0] : 1;
    bool cut[TN_PROGRAM_MAX_INPUTS];
    bool any_cut = false;
    for (int k = 0; k < n_inputs; ++k) {
        cut[k] = dst->rank >= 2 && inputs[k]->rank == dst->rank && (int64_t)inputs[k]->shape.sizes[0] == rows && rows > 1;
        any_cut = any_cut || cut[k];
        TN_TRY(grow(&p.stage_in[k], &p.stage_in_bytes[k], inputs[k]->size * es));
    }
    TN_TRY(grow(&p.stage_out, &p.stage_out_bytes, dst->size * es));
    int n = chunks > 0 ? chunks : 8;
    if (n > kMaxChunks) n = kMaxChunks;
    if (n > rows) n = (int)rows;
    if (!any_cut) n = 1;

    tn_tensor_t dev_in[TN_PROGRAM_MAX_INPUTS];
    for (int k = 0; k < n_inputs; ++k) {
        dev_in[k] = *inputs[k];
        dev_in[k].address = p.stage_in[k];
        dev_in[k].environment.kind = TN_DEVICE;
        dev_in[k].environment.resource.device.id = device->id;
        if (!cut[k]) TN_CUDA(cudaMemcpyAsync(p.stage_in[k], inputs[k]->address, inputs[k]->size * es, cudaMemcpyHostToDevice, p.in));
    }
    tn_tensor_t dev_out = *dst;
    dev_out.address = p.stage_out;
    dev_out.environment.kind = TN_DEVICE;
    dev_out.environment.resource.device.id = device->id;
    const size_t out_row_bytes = (dst->size / (size_t)rows) * es;

    tn_status st = TN_SUCCESS;
    for (int c = 0; c < n && st == TN_SUCCESS; ++c) {
        const int64_t lo = rows * c / n, hi = rows * (c + 1) / n;
        if (hi == lo) continue;
        tn_tensor_t views[TN_PROGRAM_MAX_INPUTS];
        const tn_tensor_t* view_ptrs[TN_PROGRAM_MAX_INPUTS];
        for (int k = 0; k < n_inputs; ++k) {
            views[k] = dev_in[k];
            if (cut[k]) {
                const size_t row_bytes = (inputs[k]->size / (size_t)rows) * es;
                views[k].address = static_cast<uint8_t*>(p.stage_in[k]) + (size_t)lo * row_bytes;
                views[k].shape.sizes[0] = (size_t)(hi - lo);
                views[k].size = (inputs[k]->size / (size_t)rows) * (size_t)(hi - lo);
                TN_CUDA(cudaMemcpyAsync(views[k].address, static_cast<const uint8_t*>(inputs[k]->address) + (size_t)lo * row_bytes,
                                        (size_t)(hi - lo) * row_bytes, cudaMemcpyHostToDevice, p.in));
            }
            view_ptrs[k] = &views[k];
        }
        TN_CUDA(cudaEventRecord(p.arrived[c], p.in));
        TN_CUDA(cudaStreamWaitEvent(p.run, p.arrived[c], 0));
        tn_tensor_t out_view = dev_out;
        if (any_cut) {
            out_view.address = static_cast<uint8_t*>(p.stage_out) + (size_t)lo * out_row_bytes;
            out_view.shape.sizes[0] = (size_t)(hi - lo);
            out_view.size = (dst->size / (size_t)rows) * (size_t)(hi - lo);
        }
        tn_stream_t run_stream;
        run_stream.address = reinterpret_cast<uintptr_t>(p.run);
        st = tn_eltwise_program(view_ptrs, n_inputs, nodes, n_nodes, &out_view, run_stream);
        if (st != TN_SUCCESS) break;
        TN_CUDA(cudaEventRecord(p.done[c], p.run));
        TN_CUDA(cudaStreamWaitEvent(p.out, p.done[c], 0));
        TN_CUDA(cudaMemcpyAsync(static_cast<uint8_t*>(dst->address) + (any_cut ? (size_t)lo * out_row_bytes : 0), out_view.address,
                                out_view.size * es, cudaMemcpyDeviceToHost, p.out));
    }
    // the call returns when the result is complete in host memory (and the staging buffers are idle)
    const cudaError_t e1 = cudaStreamSynchronize(p.out), e2 = cudaStreamSynchronize(p.run), e3 = cudaStreamSynchronize(p.in);
    if (st != TN_SUCCESS) return st;
    if (e1 != cudaSuccess || e2 != cudaSuccess || e3 != cudaSuccess)
        return fail(TN_ERROR, "host pipeline failed: %s", cudaGetErrorString(e1 != cudaSuccess ? e1 : e2 != cudaSuccess ? e2 : e3));
    return TN_SUCCESS;
}

}  // extern "C"

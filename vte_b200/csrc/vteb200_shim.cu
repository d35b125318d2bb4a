// libvteb200.so: flat C ABI over the CUDA runtime (linked statically) and the
// CUDA driver (entry points resolved at run time through the runtime, so the
// library loads on a machine without a driver), plus direct launchers for the
// decode-attention kernels.  Declarations and the reference interfaces they
// replace are in include/vteb200.h.
#include <cuda.h>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "../../include/vteb200.h"
#include "kernels/decode_attention.cu"
#include "kernels/aux_kernels.cu"

namespace {

thread_local char g_err[512] = "";
bool g_initialized = false;
int g_device = -1;

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int check_rt(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return 0;
    snprintf(g_err, sizeof(g_err), "%s: %s (%d)", what, cudaGetErrorString(e), (int)e);
    return (int)e;
}

// ---- driver entry points, resolved lazily --------------------------------
struct DriverApi {
    CUresult (*ModuleLoad)(CUmodule*, const char*) = nullptr;
    CUresult (*ModuleGetFunction)(CUfunction*, CUmodule, const char*) = nullptr;
    CUresult (*ModuleUnload)(CUmodule) = nullptr;
    CUresult (*FuncSetAttribute)(CUfunction, CUfunction_attribute, int) = nullptr;
    CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned,
                             unsigned, CUstream, void**, void**) = nullptr;
    CUresult (*LaunchKernelEx)(const CUlaunchConfig*, CUfunction, void**, void**) = nullptr;
    CUresult (*GetErrorString)(CUresult, const char**) = nullptr;
    CUresult (*TensorMapEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                     const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                     CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill) = nullptr;
    bool ready = false;
} g_drv;

template <typename F>
int resolve(const char* name, F* out) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || fn == nullptr || q != cudaDriverEntryPointSuccess) {
        cudaGetLastError();
        return fail(VTEB_ERR_DRIVER_ENTRY, "driver entry point %s not available", name);
    }
    *out = reinterpret_cast<F>(fn);
    return 0;
}

int driver_api() {
    if (g_drv.ready) return 0;
    int rc;
    if ((rc = resolve("cuModuleLoad", &g_drv.ModuleLoad))) return rc;
    if ((rc = resolve("cuModuleGetFunction", &g_drv.ModuleGetFunction))) return rc;
    if ((rc = resolve("cuModuleUnload", &g_drv.ModuleUnload))) return rc;
    if ((rc = resolve("cuFuncSetAttribute", &g_drv.FuncSetAttribute))) return rc;
    if ((rc = resolve("cuLaunchKernel", &g_drv.LaunchKernel))) return rc;
    if ((rc = resolve("cuLaunchKernelEx", &g_drv.LaunchKernelEx))) return rc;
    if ((rc = resolve("cuGetErrorString", &g_drv.GetErrorString))) return rc;
    if ((rc = resolve("cuTensorMapEncodeTiled", &g_drv.TensorMapEncodeTiled))) return rc;
    g_drv.ready = true;
    return 0;
}

int check_drv(CUresult r, const char* what) {
    if (r == CUDA_SUCCESS) return 0;
    const char* s = nullptr;
    if (g_drv.GetErrorString) g_drv.GetErrorString(r, &s);
    snprintf(g_err, sizeof(g_err), "%s: %s (%d)", what, s ? s : "unknown driver error", (int)r);
    return (int)r;
}

#define REQUIRE_INIT() \
    do { if (!g_initialized) return fail(VTEB_ERR_NOT_INITIALIZED, "vteb_init has not been called"); } while (0)

// ---- NCCL through dlopen ---------------------------------------------------
struct Id128 { char bytes[128]; };
struct NcclFns {
    void* lib = nullptr;
    int (*GetUniqueId)(Id128*) = nullptr;
    int (*CommInitRank)(void**, int, Id128, int) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    int (*CommDestroy)(void*) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
} g_nccl;

constexpr int kNcclFloat32 = 7;   // ncclFloat32
constexpr int kNcclMax = 2;       // ncclMax

int nccl_api() {
    if (g_nccl.lib) return 0;
    const char* override_path = getenv("VTEB_NCCL_LIBRARY");
    void* lib = nullptr;
    if (override_path && *override_path) lib = dlopen(override_path, RTLD_NOW | RTLD_LOCAL);
    if (!lib) lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
    if (!lib) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
    if (!lib) return fail(VTEB_ERR_NCCL_UNAVAILABLE, "cannot open libnccl.so.2: %s", dlerror());
    NcclFns f;
    f.lib = lib;
    f.GetUniqueId = reinterpret_cast<decltype(f.GetUniqueId)>(dlsym(lib, "ncclGetUniqueId"));
    f.CommInitRank = reinterpret_cast<decltype(f.CommInitRank)>(dlsym(lib, "ncclCommInitRank"));
    f.AllGather = reinterpret_cast<decltype(f.AllGather)>(dlsym(lib, "ncclAllGather"));
    f.AllReduce = reinterpret_cast<decltype(f.AllReduce)>(dlsym(lib, "ncclAllReduce"));
    f.CommDestroy = reinterpret_cast<decltype(f.CommDestroy)>(dlsym(lib, "ncclCommDestroy"));
    f.GetErrorString = reinterpret_cast<decltype(f.GetErrorString)>(dlsym(lib, "ncclGetErrorString"));
    if (!f.GetUniqueId || !f.CommInitRank || !f.AllGather || !f.AllReduce || !f.CommDestroy)
        return fail(VTEB_ERR_NCCL_UNAVAILABLE, "libnccl is missing a required symbol");
    g_nccl = f;
    return 0;
}

int check_nccl(int r, const char* what) {
    if (r == 0) return 0;
    const char* s = g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "nccl error";
    snprintf(g_err, sizeof(g_err), "%s: %s (%d)", what, s, r);
    return r;
}

// Per-process record of which in-library kernels already had their dynamic
// shared memory limit raised.
bool g_fast_attr_set[7] = {false, false, false, false, false, false, false};

// Tensor map over a K or V cache seen as a matrix of `n_rows` position rows of `row_halves`
// fp16 values: boxes of 64 halves x `box_rows` rows, 128-byte swizzle.
int encode_kv_tensor_map(vteb::KvTensorMap* out, const void* cache, unsigned long long n_rows, int row_halves,
                         int box_rows) {
    static_assert(sizeof(vteb::KvTensorMap) == sizeof(CUtensorMap), "tensor map size");
    int rc = driver_api();
    if (rc) return rc;
    if (!out || !cache || ((uintptr_t)cache & 15) || n_rows == 0 || n_rows > 0xffffffffULL || row_halves < 64 ||
        row_halves % 64 || box_rows < 1 || box_rows > 256)
        return fail(VTEB_ERR_INVALID_ARGUMENT, "tensor map: cache %p rows %llu row_halves %d box_rows %d", cache,
                    n_rows, row_halves, box_rows);
    const cuuint64_t dims[2] = {(cuuint64_t)row_halves, (cuuint64_t)n_rows};
    const cuuint64_t strides[1] = {(cuuint64_t)row_halves * 2};
    const cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    const cuuint32_t elem_strides[2] = {1u, 1u};
    return check_drv(g_drv.TensorMapEncodeTiled(reinterpret_cast<CUtensorMap*>(out), CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                                                const_cast<void*>(cache), dims, strides, box, elem_strides,
                                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE),
                     "cuTensorMapEncodeTiled");
}

template <typename... Args>
int launch_rt(void (*kernel)(Args...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
              bool programmatic, Args... args) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (programmatic) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    return check_rt(cudaLaunchKernelEx(&cfg, kernel, args...), "cudaLaunchKernelEx");
}

}  // namespace

extern "C" {

const char* vteb_last_error_string(void) { return g_err; }
int vteb_version(void) { return 100; }

// ---- device ---------------------------------------------------------------
int vteb_device_count(int* count) {
    if (!count) return fail(VTEB_ERR_INVALID_ARGUMENT, "count is null");
    return check_rt(cudaGetDeviceCount(count), "cudaGetDeviceCount");
}

int vteb_init(int device_index) {
    int n = 0;
    int rc = check_rt(cudaGetDeviceCount(&n), "cudaGetDeviceCount");
    if (rc) return rc;
    if (device_index < 0 || device_index >= n)
        return fail(VTEB_ERR_INVALID_ARGUMENT, "device %d out of range (0..%d)", device_index, n - 1);
    if ((rc = check_rt(cudaSetDevice(device_index), "cudaSetDevice"))) return rc;
    if ((rc = check_rt(cudaFree(nullptr), "context creation"))) return rc;
    if ((rc = driver_api())) return rc;
    g_device = device_index;
    g_initialized = true;
    return 0;
}

int vteb_current_device(int* device_index) {
    REQUIRE_INIT();
    if (!device_index) return fail(VTEB_ERR_INVALID_ARGUMENT, "device_index is null");
    *device_index = g_device;
    return 0;
}

int vteb_device_attr(int device_index, int attr_id, int* value) {
    if (!value) return fail(VTEB_ERR_INVALID_ARGUMENT, "value is null");
    cudaDeviceAttr a;
    switch (attr_id) {
    case VTEB_ATTR_SM_COUNT: a = cudaDevAttrMultiProcessorCount; break;
    case VTEB_ATTR_MAX_THREADS_PER_BLOCK: a = cudaDevAttrMaxThreadsPerBlock; break;
    case VTEB_ATTR_MAX_SMEM_PER_BLOCK: a = cudaDevAttrMaxSharedMemoryPerBlock; break;
    case VTEB_ATTR_MAX_SMEM_PER_BLOCK_OPTIN: a = cudaDevAttrMaxSharedMemoryPerBlockOptin; break;
    case VTEB_ATTR_CC_MAJOR: a = cudaDevAttrComputeCapabilityMajor; break;
    case VTEB_ATTR_CC_MINOR: a = cudaDevAttrComputeCapabilityMinor; break;
    case VTEB_ATTR_L2_BYTES: a = cudaDevAttrL2CacheSize; break;
    case VTEB_ATTR_CLOCK_KHZ: a = cudaDevAttrClockRate; break;
    default: return fail(VTEB_ERR_INVALID_ARGUMENT, "unknown attribute id %d", attr_id);
    }
    return check_rt(cudaDeviceGetAttribute(value, a, device_index), "cudaDeviceGetAttribute");
}

int vteb_device_name(int device_index, char* buf, int buf_len) {
    if (!buf || buf_len <= 0) return fail(VTEB_ERR_INVALID_ARGUMENT, "bad name buffer");
    cudaDeviceProp prop;
    int rc = check_rt(cudaGetDeviceProperties(&prop, device_index), "cudaGetDeviceProperties");
    if (rc) return rc;
    snprintf(buf, (size_t)buf_len, "%s", prop.name);
    return 0;
}

int vteb_mem_info(size_t* free_bytes, size_t* total_bytes) {
    REQUIRE_INIT();
    if (!free_bytes || !total_bytes) return fail(VTEB_ERR_INVALID_ARGUMENT, "null output");
    return check_rt(cudaMemGetInfo(free_bytes, total_bytes), "cudaMemGetInfo");
}

int vteb_device_synchronize(void) {
    REQUIRE_INIT();
    return check_rt(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
}

// ---- memory ---------------------------------------------------------------
int vteb_malloc(void** dev_ptr, size_t bytes) {
    REQUIRE_INIT();
    if (!dev_ptr || bytes == 0) return fail(VTEB_ERR_INVALID_ARGUMENT, "malloc of %zu bytes", bytes);
    return check_rt(cudaMalloc(dev_ptr, bytes), "cudaMalloc");
}

int vteb_free(void* dev_ptr) {
    REQUIRE_INIT();
    return check_rt(cudaFree(dev_ptr), "cudaFree");
}

int vteb_memcpy_h2d(void* dst, const void* src, size_t bytes) {
    REQUIRE_INIT();
    if (!dst || !src) return fail(VTEB_ERR_INVALID_ARGUMENT, "null pointer in h2d copy");
    return check_rt(cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice), "cudaMemcpy (H2D)");
}

int vteb_memcpy_d2h(void* dst, const void* src, size_t bytes) {
    REQUIRE_INIT();
    if (!dst || !src) return fail(VTEB_ERR_INVALID_ARGUMENT, "null pointer in d2h copy");
    return check_rt(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost), "cudaMemcpy (D2H)");
}

int vteb_memcpy_d2d(void* dst, const void* src, size_t bytes) {
    REQUIRE_INIT();
    if (!dst || !src) return fail(VTEB_ERR_INVALID_ARGUMENT, "null pointer in d2d copy");
    return check_rt(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToDevice), "cudaMemcpy (D2D)");
}

int vteb_memcpy_h2d_async(void* dst, const void* src, size_t bytes, void* stream) {
    REQUIRE_INIT();
    if (!dst || !src) return fail(VTEB_ERR_INVALID_ARGUMENT, "null pointer in async h2d copy");
    return check_rt(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream),
                    "cudaMemcpyAsync (H2D)");
}

int vteb_memcpy_d2h_async(void* dst, const void* src, size_t bytes, void* stream) {
    REQUIRE_INIT();
    if (!dst || !src) return fail(VTEB_ERR_INVALID_ARGUMENT, "null pointer in async d2h copy");
    return check_rt(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream),
                    "cudaMemcpyAsync (D2H)");
}

int vteb_memset(void* dst, int value, size_t bytes) {
    REQUIRE_INIT();
    if (!dst) return fail(VTEB_ERR_INVALID_ARGUMENT, "null pointer in memset");
    return check_rt(cudaMemset(dst, value, bytes), "cudaMemset");
}

int vteb_memset_async(void* dst, int value, size_t bytes, void* stream) {
    REQUIRE_INIT();
    if (!dst) return fail(VTEB_ERR_INVALID_ARGUMENT, "null pointer in memset");
    return check_rt(cudaMemsetAsync(dst, value, bytes, (cudaStream_t)stream), "cudaMemsetAsync");
}

int vteb_host_alloc(void** host_ptr, size_t bytes) {
    REQUIRE_INIT();
    if (!host_ptr || bytes == 0) return fail(VTEB_ERR_INVALID_ARGUMENT, "host alloc of %zu bytes", bytes);
    return check_rt(cudaHostAlloc(host_ptr, bytes, cudaHostAllocDefault), "cudaHostAlloc");
}

int vteb_host_free(void* host_ptr) {
    REQUIRE_INIT();
    return check_rt(cudaFreeHost(host_ptr), "cudaFreeHost");
}

// ---- modules and launches -------------------------------------------------
int vteb_module_load(void** module, const char* cubin_path) {
    REQUIRE_INIT();
    if (!module || !cubin_path) return fail(VTEB_ERR_INVALID_ARGUMENT, "null module or path");
    CUmodule m = nullptr;
    int rc = check_drv(g_drv.ModuleLoad(&m, cubin_path), "cuModuleLoad");
    if (rc) return rc;
    *module = m;
    return 0;
}

int vteb_module_get_function(void** function, void* module, const char* name) {
    REQUIRE_INIT();
    if (!function || !module || !name) return fail(VTEB_ERR_INVALID_ARGUMENT, "null argument");
    CUfunction f = nullptr;
    int rc = check_drv(g_drv.ModuleGetFunction(&f, (CUmodule)module, name), "cuModuleGetFunction");
    if (rc) return rc;
    *function = f;
    return 0;
}

int vteb_module_unload(void* module) {
    REQUIRE_INIT();
    if (!module) return fail(VTEB_ERR_INVALID_ARGUMENT, "null module");
    return check_drv(g_drv.ModuleUnload((CUmodule)module), "cuModuleUnload");
}

int vteb_func_set_max_dynamic_smem(void* function, int bytes) {
    REQUIRE_INIT();
    if (!function || bytes < 0) return fail(VTEB_ERR_INVALID_ARGUMENT, "bad function or size");
    return check_drv(g_drv.FuncSetAttribute((CUfunction)function,
                                            CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, bytes),
                     "cuFuncSetAttribute(max dynamic shared memory)");
}

int vteb_func_set_shared_carveout(void* function, int percent) {
    REQUIRE_INIT();
    if (!function || percent < 0 || percent > 100) return fail(VTEB_ERR_INVALID_ARGUMENT, "bad function or percent");
    return check_drv(g_drv.FuncSetAttribute((CUfunction)function,
                                            CU_FUNC_ATTRIBUTE_PREFERRED_SHARED_MEMORY_CARVEOUT, percent),
                     "cuFuncSetAttribute(shared memory carve-out)");
}

int vteb_launch(void* function, unsigned gx, unsigned gy, unsigned gz, unsigned bx, unsigned by,
                unsigned bz, unsigned shared_mem_bytes, void* stream, void** params, unsigned flags) {
    REQUIRE_INIT();
    if (!function) return fail(VTEB_ERR_INVALID_ARGUMENT, "null function");
    if (!gx || !gy || !gz || !bx || !by || !bz) return fail(VTEB_ERR_INVALID_ARGUMENT, "zero launch dimension");
    if (flags & VTEB_LAUNCH_PROGRAMMATIC) {
        CUlaunchConfig cfg;
        memset(&cfg, 0, sizeof(cfg));
        cfg.gridDimX = gx; cfg.gridDimY = gy; cfg.gridDimZ = gz;
        cfg.blockDimX = bx; cfg.blockDimY = by; cfg.blockDimZ = bz;
        cfg.sharedMemBytes = shared_mem_bytes;
        cfg.hStream = (CUstream)stream;
        CUlaunchAttribute attr;
        memset(&attr, 0, sizeof(attr));
        attr.id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
        attr.value.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        return check_drv(g_drv.LaunchKernelEx(&cfg, (CUfunction)function, params, nullptr), "cuLaunchKernelEx");
    }
    return check_drv(g_drv.LaunchKernel((CUfunction)function, gx, gy, gz, bx, by, bz, shared_mem_bytes,
                                        (CUstream)stream, params, nullptr),
                     "cuLaunchKernel");
}

// ---- streams, events, graphs ----------------------------------------------
int vteb_stream_create(void** stream) {
    REQUIRE_INIT();
    if (!stream) return fail(VTEB_ERR_INVALID_ARGUMENT, "null stream output");
    cudaStream_t s;
    int rc = check_rt(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking), "cudaStreamCreate");
    if (rc) return rc;
    *stream = s;
    return 0;
}

int vteb_stream_destroy(void* stream) {
    REQUIRE_INIT();
    return check_rt(cudaStreamDestroy((cudaStream_t)stream), "cudaStreamDestroy");
}

int vteb_stream_synchronize(void* stream) {
    REQUIRE_INIT();
    return check_rt(cudaStreamSynchronize((cudaStream_t)stream), "cudaStreamSynchronize");
}

int vteb_stream_begin_capture(void* stream, int mode) {
    REQUIRE_INIT();
    cudaStreamCaptureMode m = mode == 0 ? cudaStreamCaptureModeGlobal
                            : mode == 1 ? cudaStreamCaptureModeThreadLocal
                                        : cudaStreamCaptureModeRelaxed;
    return check_rt(cudaStreamBeginCapture((cudaStream_t)stream, m), "cudaStreamBeginCapture");
}

int vteb_stream_end_capture(void* stream, void** graph) {
    REQUIRE_INIT();
    if (!graph) return fail(VTEB_ERR_INVALID_ARGUMENT, "null graph output");
    cudaGraph_t g = nullptr;
    int rc = check_rt(cudaStreamEndCapture((cudaStream_t)stream, &g), "cudaStreamEndCapture");
    if (rc) return rc;
    *graph = g;
    return 0;
}

int vteb_graph_instantiate(void** graph_exec, void* graph) {
    REQUIRE_INIT();
    if (!graph_exec || !graph) return fail(VTEB_ERR_INVALID_ARGUMENT, "null graph argument");
    cudaGraphExec_t e = nullptr;
    int rc = check_rt(cudaGraphInstantiate(&e, (cudaGraph_t)graph, 0), "cudaGraphInstantiate");
    if (rc) return rc;
    *graph_exec = e;
    return 0;
}

int vteb_graph_launch(void* graph_exec, void* stream) {
    REQUIRE_INIT();
    if (!graph_exec) return fail(VTEB_ERR_INVALID_ARGUMENT, "null graph exec");
    return check_rt(cudaGraphLaunch((cudaGraphExec_t)graph_exec, (cudaStream_t)stream), "cudaGraphLaunch");
}

int vteb_graph_destroy(void* graph) {
    REQUIRE_INIT();
    return check_rt(cudaGraphDestroy((cudaGraph_t)graph), "cudaGraphDestroy");
}

int vteb_graph_exec_destroy(void* graph_exec) {
    REQUIRE_INIT();
    return check_rt(cudaGraphExecDestroy((cudaGraphExec_t)graph_exec), "cudaGraphExecDestroy");
}

int vteb_graph_node_count(void* graph, size_t* count) {
    REQUIRE_INIT();
    if (!graph || !count) return fail(VTEB_ERR_INVALID_ARGUMENT, "null graph argument");
    return check_rt(cudaGraphGetNodes((cudaGraph_t)graph, nullptr, count), "cudaGraphGetNodes");
}

int vteb_event_create(void** event) {
    REQUIRE_INIT();
    if (!event) return fail(VTEB_ERR_INVALID_ARGUMENT, "null event output");
    cudaEvent_t e;
    int rc = check_rt(cudaEventCreate(&e), "cudaEventCreate");
    if (rc) return rc;
    *event = e;
    return 0;
}

int vteb_event_record(void* event, void* stream) {
    REQUIRE_INIT();
    return check_rt(cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream), "cudaEventRecord");
}

int vteb_event_synchronize(void* event) {
    REQUIRE_INIT();
    return check_rt(cudaEventSynchronize((cudaEvent_t)event), "cudaEventSynchronize");
}

int vteb_event_elapsed_ms(float* ms, void* start, void* stop) {
    REQUIRE_INIT();
    if (!ms) return fail(VTEB_ERR_INVALID_ARGUMENT, "null ms output");
    return check_rt(cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)stop), "cudaEventElapsedTime");
}

int vteb_event_destroy(void* event) {
    REQUIRE_INIT();
    return check_rt(cudaEventDestroy((cudaEvent_t)event), "cudaEventDestroy");
}

// ---- NCCL -------------------------------------------------------------------
int vteb_nccl_unique_id(void* id128) {
    if (!id128) return fail(VTEB_ERR_INVALID_ARGUMENT, "null id buffer");
    int rc = nccl_api();
    if (rc) return rc;
    return check_nccl(g_nccl.GetUniqueId(reinterpret_cast<Id128*>(id128)), "ncclGetUniqueId");
}

int vteb_nccl_comm_init_rank(void** comm, int n_ranks, const void* id128, int rank) {
    REQUIRE_INIT();
    if (!comm || !id128 || n_ranks <= 0 || rank < 0 || rank >= n_ranks)
        return fail(VTEB_ERR_INVALID_ARGUMENT, "bad communicator arguments");
    int rc = nccl_api();
    if (rc) return rc;
    Id128 id;
    memcpy(&id, id128, sizeof(id));
    return check_nccl(g_nccl.CommInitRank(comm, n_ranks, id, rank), "ncclCommInitRank");
}

int vteb_nccl_all_gather_f32(void* comm, const void* send, void* recv, size_t count_per_rank, void* stream) {
    REQUIRE_INIT();
    if (!comm || !send || !recv) return fail(VTEB_ERR_INVALID_ARGUMENT, "null allgather argument");
    return check_nccl(g_nccl.AllGather(send, recv, count_per_rank, kNcclFloat32, comm, (cudaStream_t)stream),
                      "ncclAllGather");
}

int vteb_nccl_all_reduce_max_f32(void* comm, const void* send, void* recv, size_t count, void* stream) {
    REQUIRE_INIT();
    if (!comm || !send || !recv) return fail(VTEB_ERR_INVALID_ARGUMENT, "null allreduce argument");
    return check_nccl(g_nccl.AllReduce(send, recv, count, kNcclFloat32, kNcclMax, comm, (cudaStream_t)stream),
                      "ncclAllReduce");
}

int vteb_nccl_comm_destroy(void* comm) {
    if (!comm) return fail(VTEB_ERR_INVALID_ARGUMENT, "null communicator");
    if (!g_nccl.lib) return fail(VTEB_ERR_NCCL_UNAVAILABLE, "nccl was never opened");
    return check_nccl(g_nccl.CommDestroy(comm), "ncclCommDestroy");
}

// ---- peer memory ---------------------------------------------------------------
int vteb_ipc_get_handle(void* dev_ptr, void* handle64) {
    REQUIRE_INIT();
    if (!dev_ptr || !handle64) return fail(VTEB_ERR_INVALID_ARGUMENT, "null ipc argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "ipc handle size");
    cudaIpcMemHandle_t h;
    int rc = check_rt(cudaIpcGetMemHandle(&h, dev_ptr), "cudaIpcGetMemHandle");
    if (rc) return rc;
    memcpy(handle64, &h, sizeof(h));
    return 0;
}

int vteb_ipc_open_handle(const void* handle64, void** dev_ptr) {
    REQUIRE_INIT();
    if (!dev_ptr || !handle64) return fail(VTEB_ERR_INVALID_ARGUMENT, "null ipc argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    return check_rt(cudaIpcOpenMemHandle(dev_ptr, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
}

int vteb_ipc_close_handle(void* dev_ptr) {
    REQUIRE_INIT();
    if (!dev_ptr) return fail(VTEB_ERR_INVALID_ARGUMENT, "null ipc pointer");
    return check_rt(cudaIpcCloseMemHandle(dev_ptr), "cudaIpcCloseMemHandle");
}

// ---- split-KV decode attention ---------------------------------------------
static int fill_plan(int num_q_heads, int num_kv_heads, int head_dim, int compact, vteb_fast_plan* plan) {
    if (!plan) return fail(VTEB_ERR_INVALID_ARGUMENT, "null plan");
    const vteb::FastPlan p = vteb::make_fast_plan(num_q_heads, num_kv_heads, head_dim, compact);
    memset(plan, 0, sizeof(*plan));
    plan->ok = p.ok;
    plan->hg = p.hg;
    plan->n_hgroups = p.n_hgroups;
    plan->tile = p.tile;
    plan->nstages = p.nstages;
    plan->smem_bytes = p.smem_bytes;
    plan->threads = p.threads;
    plan->combine_dsplit = head_dim >= 32 ? head_dim / 32 : 1;   // one CTA per 32 output columns
    plan->combine_smem_bytes = 4;
    return 0;
}

int vteb_split_kv_plan(int num_q_heads, int num_kv_heads, int head_dim, vteb_fast_plan* plan) {
    return fill_plan(num_q_heads, num_kv_heads, head_dim, 0, plan);
}

int vteb_split_kv_plan_compact(int num_q_heads, int num_kv_heads, int head_dim, vteb_fast_plan* plan) {
    return fill_plan(num_q_heads, num_kv_heads, head_dim, 1, plan);
}

int vteb_kv_tensor_map(void* out_128_bytes, const void* cache, long long n_rows, int row_halves, int box_rows) {
    REQUIRE_INIT();
    if (n_rows <= 0) return fail(VTEB_ERR_INVALID_ARGUMENT, "tensor map: %lld rows", n_rows);
    vteb::KvTensorMap tm;
    int rc = encode_kv_tensor_map(&tm, cache, (unsigned long long)n_rows, row_halves, box_rows);
    if (rc) return rc;
    memcpy(out_128_bytes, &tm, sizeof(tm));
    return 0;
}

int vteb_combine_rows_epl(int rows, int head_dim) {
    int epl = head_dim / 32;
    if (epl > 8) epl = 8;
    if (epl < 1) epl = 1;
    // halve the columns per lane until about two thousand warps exist
    while (epl > 1 && (long long)rows * (head_dim / (32 * epl)) < 2048) epl /= 2;
    return epl;
}

static int validate_attention_args(const void* q, const void* k_cache, const void* v_cache,
                                   const int* kv_offsets, void* output, int batch, int num_q_heads,
                                   int num_kv_heads, int head_dim, long long kv_batch_stride, int max_chunks) {
    if (!q || !k_cache || !v_cache || !kv_offsets || !output)
        return fail(VTEB_ERR_INVALID_ARGUMENT, "null tensor pointer");
    if (batch <= 0 || num_q_heads <= 0 || num_kv_heads <= 0 || max_chunks <= 0)
        return fail(VTEB_ERR_INVALID_ARGUMENT, "non-positive dimension");
    if (num_q_heads % num_kv_heads != 0)
        return fail(VTEB_ERR_INVALID_ARGUMENT, "num_q_heads %d is not a multiple of num_kv_heads %d",
                    num_q_heads, num_kv_heads);
    if (head_dim != 64 && head_dim != 128 && head_dim != 256)
        return fail(VTEB_ERR_UNSUPPORTED, "head_dim %d (supported: 64, 128, 256)", head_dim);
    if (kv_batch_stride < 0 || kv_batch_stride > 0x7fffffffLL)
        return fail(VTEB_ERR_INVALID_ARGUMENT, "kv_batch_stride %lld does not fit the kernel ABI's int", kv_batch_stride);
    if (((uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)q) & 15)
        return fail(VTEB_ERR_INVALID_ARGUMENT, "q, k_cache and v_cache must be 16-byte aligned");
    if (kv_batch_stride % 8 != 0)
        return fail(VTEB_ERR_INVALID_ARGUMENT, "kv_batch_stride must be a multiple of 8 elements");
    return 0;
}

int vteb_split_kv_decode(const void* q, const void* k_cache, const void* v_cache, const int* kv_offsets,
                         void* output, int out_is_f32, float* partial_m, float* partial_l,
                         float* partial_o, int* work, int batch, int num_q_heads, int num_kv_heads,
                         int head_dim, float scale, long long kv_batch_stride, int max_chunks,
                         int min_chunk, unsigned flags, int n_ctas, void* stream) {
    REQUIRE_INIT();
    int rc = validate_attention_args(q, k_cache, v_cache, kv_offsets, output, batch, num_q_heads,
                                     num_kv_heads, head_dim, kv_batch_stride, max_chunks);
    if (rc) return rc;
    if (!partial_m || !partial_l || !partial_o || !work)
        return fail(VTEB_ERR_INVALID_ARGUMENT, "null scratch pointer");
    cudaStream_t s = (cudaStream_t)stream;
    const bool pdl = (flags & VTEB_ATTN_PROGRAMMATIC) != 0;
    const __half* qh = (const __half*)q;
    const __half* kh = (const __half*)k_cache;
    const __half* vh = (const __half*)v_cache;

    if (flags & VTEB_ATTN_COMPAT) {
        rc = launch_rt(flash_attention_split_kv_partial_kernel, dim3(batch, num_q_heads, max_chunks),
                       dim3(head_dim), 0, s, pdl, qh, kh, vh, partial_m, partial_l, partial_o, num_q_heads,
                       num_kv_heads, head_dim, scale, kv_offsets, (int)kv_batch_stride, max_chunks);
        if (rc) return rc;
        if (out_is_f32)
            return launch_rt(flash_attention_split_kv_reduce_f32_kernel, dim3(batch, num_q_heads, 1),
                             dim3(head_dim), (size_t)max_chunks * 4, s, pdl, (const float*)partial_m,
                             (const float*)partial_l, (const float*)partial_o, (float*)output, num_q_heads,
                             head_dim, max_chunks);
        return launch_rt(flash_attention_split_kv_reduce_kernel, dim3(batch, num_q_heads, 1), dim3(head_dim),
                         (size_t)max_chunks * 4, s, pdl, (const float*)partial_m, (const float*)partial_l,
                         (const float*)partial_o, (__half*)output, num_q_heads, head_dim, max_chunks);
    }

    bool compact = (flags & VTEB_ATTN_COMPACT) != 0;
    vteb::FastPlan p = vteb::make_fast_plan(num_q_heads, num_kv_heads, head_dim, compact ? 1 : 0);
    if (compact && !p.ok) {   // more KV heads per group than the compact shape's consumer warps can serve
        compact = false;
        p = vteb::make_fast_plan(num_q_heads, num_kv_heads, head_dim, 0);
    }
    if (!p.ok)
        return fail(VTEB_ERR_UNSUPPORTED, "fast split kernel does not cover Hq=%d Hkv=%d D=%d; pass VTEB_ATTN_COMPAT",
                    num_q_heads, num_kv_heads, head_dim);
    const long long items = (long long)batch * p.n_hgroups * max_chunks;
    if (items > 0x7fffffffLL) return fail(VTEB_ERR_TOO_LARGE, "too many work items");
    if (n_ctas <= 0) {
        int sms = 0;
        if ((rc = check_rt(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, g_device), "sm count"))) return rc;
        n_ctas = sms;
    }
    const bool balanced = (flags & VTEB_ATTN_BALANCED) != 0;
    if (balanced && max_chunks < 2) return fail(VTEB_ERR_INVALID_ARGUMENT, "VTEB_ATTN_BALANCED needs max_chunks >= 2");
    if (balanced && compact) return fail(VTEB_ERR_INVALID_ARGUMENT, "VTEB_ATTN_BALANCED and VTEB_ATTN_COMPACT exclude each other");
    if (n_ctas > items && !balanced) n_ctas = (int)items;

    typedef void (*FastKernel)(const __half*, const __half*, const __half*, float*, float*, float*, int, int,
                               int, float, const int*, int, int, int, int, int, const int*, int*, int*, const __half*,
                               const __half*, void*, int, const vteb::KvTensorMap, const vteb::KvTensorMap);
    FastKernel fk;
    int slot;
    if (compact && head_dim == 64) { fk = vteb_split_kv_partial_compact_d64_kernel; slot = 3; }
    else if (compact && head_dim == 128 && (flags & VTEB_ATTN_SHORT_SPLITS) && max_chunks > 1) { fk = vteb_split_kv_partial_compact_cs_d128_kernel; slot = 6; }
    else if (compact && head_dim == 128) { fk = vteb_split_kv_partial_compact_d128_kernel; slot = 4; }
    else if (compact) { fk = vteb_split_kv_partial_compact_d256_kernel; slot = 5; }
    else if (head_dim == 64) { fk = vteb_split_kv_partial_d64_kernel; slot = 0; }
    else if (head_dim == 128) { fk = vteb_split_kv_partial_d128_kernel; slot = 1; }
    else { fk = vteb_split_kv_partial_d256_kernel; slot = 2; }
    if (!g_fast_attr_set[slot]) {
        if ((rc = check_rt(cudaFuncSetAttribute(fk, cudaFuncAttributeMaxDynamicSharedMemorySize, vteb::kSmemBudget),
                           "cudaFuncSetAttribute(max dynamic shared memory)"))) return rc;
        g_fast_attr_set[slot] = true;
    }
    int kflags = (flags & VTEB_ATTN_WRITE_EMPTY_O) ? kFlagWriteEmptyO : 0;
    if (balanced) kflags |= kFlagBalanced;
    // Whole tiles travel as tensor-map boxes when the caches are one matrix of position rows
    // (the stride between sequences is a whole number of rows).
    vteb::KvTensorMap tmk, tmv;
    memset(&tmk, 0, sizeof(tmk));
    memset(&tmv, 0, sizeof(tmv));
    const int row_halves = num_kv_heads * head_dim;
    if (!(flags & VTEB_ATTN_NO_TENSOR_MAPS) && kv_batch_stride % row_halves == 0 && row_halves % 64 == 0) {
        const unsigned long long rows_per_seq = (unsigned long long)(kv_batch_stride / row_halves);
        const unsigned long long n_rows = batch > 1 ? rows_per_seq * batch : 0xffffffffULL;   // one sequence: its length is not known here
        if ((rc = encode_kv_tensor_map(&tmk, k_cache, n_rows, row_halves, p.tile))) return rc;
        if ((rc = encode_kv_tensor_map(&tmv, v_cache, n_rows, row_halves, p.tile))) return rc;
        kflags |= kFlagTensorMaps;
    }
    rc = launch_rt(fk, dim3(n_ctas), dim3(p.threads), (size_t)p.smem_bytes, s, pdl, qh, kh, vh,
                   partial_m, partial_l, partial_o, num_q_heads, num_kv_heads, head_dim, scale, kv_offsets,
                   (int)kv_batch_stride, max_chunks, batch, min_chunk, kflags, (const int*)nullptr, work,
                   work + 1, (const __half*)nullptr, (const __half*)nullptr, (void*)nullptr, 0,
                   (const vteb::KvTensorMap)tmk, (const vteb::KvTensorMap)tmv);
    if (rc) return rc;

    if (max_chunks <= 32 && compact) {        // beside a compact split CTA: the small combine (64 registers), not the row kernel (111)
        const int rows = batch * num_q_heads;
        const int units = rows * (head_dim / 32);
        return launch_rt(vteb_split_kv_combine_small_kernel, dim3((units + 7) / 8), dim3(256), 0, s, pdl,
                         (const float*)partial_m, (const float*)partial_l, (const float*)partial_o, output,
                         num_q_heads, head_dim, max_chunks, out_is_f32 ? 2 : 1, work, rows, 1);
    }
    if (max_chunks <= 64 && !compact) {
        const int rows = batch * num_q_heads;
        const int epl = vteb_combine_rows_epl(rows, head_dim);
        const int units = rows * (head_dim / (32 * epl));
        return launch_rt(vteb_split_kv_combine_rows_kernel, dim3((units + 7) / 8), dim3(256), 0, s, pdl,
                         (const float*)partial_m, (const float*)partial_l, (const float*)partial_o, output,
                         num_q_heads, head_dim, max_chunks, out_is_f32 ? 2 : 1, work, rows, epl);
    }
    vteb_fast_plan hp;
    vteb_split_kv_plan(num_q_heads, num_kv_heads, head_dim, &hp);
    const int dsplit = hp.combine_dsplit;
    const size_t csmem = (size_t)(max_chunks < 256 ? max_chunks : 256) * 4;
    if (out_is_f32)
        return launch_rt(vteb_split_kv_combine_f32_kernel, dim3(batch * num_q_heads * dsplit), dim3(256), csmem,
                         s, pdl, (const float*)partial_m, (const float*)partial_l, (const float*)partial_o,
                         (float*)output, num_q_heads, head_dim, max_chunks, dsplit, work);
    return launch_rt(vteb_split_kv_combine_f16_kernel, dim3(batch * num_q_heads * dsplit), dim3(256), csmem, s,
                     pdl, (const float*)partial_m, (const float*)partial_l, (const float*)partial_o,
                     (__half*)output, num_q_heads, head_dim, max_chunks, dsplit, work);
}

// ---- the entry point that allocates nothing ---------------------------------
// Scratch for callers that may not allocate: one array per GPU that loads this
// library.  In host code `g_noalloc_scratch` is only a handle for the runtime's
// symbol lookup, never a device address; the address is resolved once per device.
static __device__ __align__(256) unsigned char g_noalloc_scratch[VTEB_NOALLOC_SCRATCH_BYTES];
static unsigned char* g_noalloc_ptr[64] = {nullptr};

int vteb_split_kv_decode_noalloc(const void* q, const void* k_cache, const void* v_cache, const int* kv_offsets,
                                 void* output, int out_is_f32, int batch, int num_q_heads, int num_kv_heads,
                                 int head_dim, float scale, long long kv_batch_stride, int max_chunks,
                                 int min_chunk, unsigned flags, int n_ctas, void* stream) {
    REQUIRE_INIT();
    if (batch <= 0 || num_q_heads <= 0 || max_chunks <= 0 || head_dim <= 0)
        return fail(VTEB_ERR_INVALID_ARGUMENT, "non-positive dimension");
    auto up = [](size_t x) { return (x + 255) / 256 * 256; };
    const size_t stats = up((size_t)batch * num_q_heads * max_chunks * 4);
    const size_t obytes = up((size_t)batch * num_q_heads * max_chunks * head_dim * 4);
    const size_t need = 256 + 2 * stats + obytes;
    if (need > VTEB_NOALLOC_SCRATCH_BYTES)
        return fail(VTEB_ERR_TOO_LARGE,
                    "vteb_split_kv_decode_noalloc: batch %d x %d heads x %d splits x head_dim %d needs %zu bytes of scratch, "
                    "the built-in array holds %u; use fewer splits or vteb_split_kv_decode with caller scratch",
                    batch, num_q_heads, max_chunks, head_dim, need, (unsigned)VTEB_NOALLOC_SCRATCH_BYTES);
    if (g_device < 0 || g_device >= 64) return fail(VTEB_ERR_UNSUPPORTED, "device index %d not supported", g_device);
    if (g_noalloc_ptr[g_device] == nullptr) {
        // one-time set-up on this device (which vteb_init made current)
        void* p = nullptr;
        int rc = check_rt(cudaGetSymbolAddress(&p, g_noalloc_scratch), "cudaGetSymbolAddress(scratch)");
        if (rc) return rc;
        if (p == nullptr) return fail(VTEB_ERR_DRIVER_ENTRY, "scratch symbol resolved to a null address");
        g_noalloc_ptr[g_device] = static_cast<unsigned char*>(p);
    }
    unsigned char* base = g_noalloc_ptr[g_device];
    int* work = reinterpret_cast<int*>(base);
    float* pm = reinterpret_cast<float*>(base + 256);
    float* pl = reinterpret_cast<float*>(base + 256 + stats);
    float* po = reinterpret_cast<float*>(base + 256 + 2 * stats);
    // the work-queue ticket must start at zero; the status word next to it keeps what an earlier
    // call may have recorded until vteb_noalloc_check_status reads it
    int rc = check_rt(cudaMemsetAsync(work, 0, 4, (cudaStream_t)stream), "scratch clear");
    if (rc) return rc;
    return vteb_split_kv_decode(q, k_cache, v_cache, kv_offsets, output, out_is_f32, pm, pl, po, work, batch,
                                num_q_heads, num_kv_heads, head_dim, scale, kv_batch_stride, max_chunks, min_chunk,
                                flags, n_ctas, stream);
}

int vteb_kv_cache_append(const void* k, const void* v, void* k_cache, void* v_cache, const int* kv_offsets,
                         int batch, int num_kv_heads, int head_dim, long long kv_batch_stride, void* stream) {
    REQUIRE_INIT();
    if (!k || !v || !k_cache || !v_cache || !kv_offsets) return fail(VTEB_ERR_INVALID_ARGUMENT, "null pointer");
    if (batch <= 0 || num_kv_heads <= 0 || head_dim <= 0 || head_dim > 1024)
        return fail(VTEB_ERR_INVALID_ARGUMENT, "bad dimension");
    if (kv_batch_stride < 0 || kv_batch_stride > 0x7fffffffLL)
        return fail(VTEB_ERR_INVALID_ARGUMENT, "kv_batch_stride does not fit the kernel ABI's int");
    return launch_rt(kv_cache_append_kernel, dim3(batch, num_kv_heads, 1), dim3(head_dim), 0,
                     (cudaStream_t)stream, false, (const __half*)k, (const __half*)v, (__half*)k_cache,
                     (__half*)v_cache, num_kv_heads, head_dim, kv_offsets, (int)kv_batch_stride);
}

int vteb_check_status(int* work, void* stream) {
    REQUIRE_INIT();
    if (!work) return fail(VTEB_ERR_INVALID_ARGUMENT, "null work pointer");
    int status = 0;
    int rc = check_rt(cudaMemcpyAsync(&status, work + 1, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream),
                      "status read");
    if (rc) return rc;
    if ((rc = check_rt(cudaStreamSynchronize((cudaStream_t)stream), "status sync"))) return rc;
    if (status != 0) {
        cudaMemsetAsync(work + 1, 0, sizeof(int), (cudaStream_t)stream);
        return fail(VTEB_ERR_DEVICE_STATUS, "a kernel gave up on a bounded wait (code %d: %s)", status,
                    status == 1 ? "a tile never arrived" : status == 2 ? "a stage was never released"
                    : status == 3 ? "the merge barrier never completed"
                                  : "another CTA or another rank never arrived");
    }
    return 0;
}

int vteb_noalloc_check_status(void* stream) {
    REQUIRE_INIT();
    if (g_device < 0 || g_device >= 64) return fail(VTEB_ERR_UNSUPPORTED, "device index %d not supported", g_device);
    if (g_noalloc_ptr[g_device] == nullptr) return 0;     // no call has used the array on this device yet
    return vteb_check_status(reinterpret_cast<int*>(g_noalloc_ptr[g_device]), stream);
}

int vteb_fill_normal_f16(void* dst, size_t n, unsigned long long seed, float sigma, float outlier_prob,
                         float outlier_scale, void* stream) {
    REQUIRE_INIT();
    if (!dst || n == 0) return fail(VTEB_ERR_INVALID_ARGUMENT, "empty fill");
    if ((uintptr_t)dst & 3) return fail(VTEB_ERR_INVALID_ARGUMENT, "fill destination must be 4-byte aligned");
    vteb_fill_normal_f16_kernel<<<148 * 8, 256, 0, (cudaStream_t)stream>>>(
        (__half*)dst, (unsigned long long)n, seed, sigma, outlier_prob, outlier_scale);
    return check_rt(cudaGetLastError(), "fill launch");
}

int vteb_read_bandwidth_probe(const void* src, size_t bytes, unsigned* sink, int n_ctas, void* stream) {
    REQUIRE_INIT();
    if (!src || !sink || bytes < 16 || n_ctas <= 0) return fail(VTEB_ERR_INVALID_ARGUMENT, "bad probe arguments");
    if ((uintptr_t)src & 15) return fail(VTEB_ERR_INVALID_ARGUMENT, "probe source must be 16-byte aligned");
    vteb_read_bandwidth_kernel<<<n_ctas, 512, 0, (cudaStream_t)stream>>>(
        (const uint4*)src, (unsigned long long)(bytes / 16), sink);
    return check_rt(cudaGetLastError(), "probe launch");
}

}  // extern "C"

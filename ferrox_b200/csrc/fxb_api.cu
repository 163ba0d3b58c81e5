// Context management and error reporting of the C ABI.
#include "fxb_common.cuh"

using namespace fxb;

namespace fxb {
thread_local std::string g_tls_error;
}

extern "C" int fxb_version(void) { return 120; }

namespace fxb {
// Self-test of the bounded-wait convention every kernel of the library follows: one warp waits on an
// mbarrier that nobody ever arrives on (no copy and no MMA is in flight, no TMEM is held).  When the
// cycle limit runs out the wait records its tag in the status block and the kernel returns normally.
constexpr int SELFTEST_WAIT_TAG = 99;
__global__ void __launch_bounds__(32) bounded_wait_selftest_kernel(DeviceStatus* status, long long limit_cycles, int* gave_up) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        mbar_init_fence();
    }
    __syncwarp();
    if (threadIdx.x == 0) {
        const bool done = mbar_wait_bounded(smem_u32(&bar), 0u, &abort_flag, status, SELFTEST_WAIT_TAG, limit_cycles);
        *gave_up = done ? 0 : 1;
    }
}
}  // namespace fxb

extern "C" int fxb_selftest_bounded_wait(fxb_handle_t h, int64_t limit_cycles, fxb_stream_t stream) {
    if (h == nullptr) return fail(nullptr, FXB_ERR_INVALID_ARGUMENT, "null ferrox_b200 handle");
    Context* c = reinterpret_cast<Context*>(h);
    FXB_CHECK_ARG(c, limit_cycles > 0 && limit_cycles <= 100000000LL, "fxb_selftest_bounded_wait: limit must be in (0, 1e8] cycles");
    // the flag lives in the handle's scratch block, past the loss kernel's counter and partial sums
    int* gave_up = reinterpret_cast<int*>(static_cast<char*>(c->d_scratch) + 8192 - 64);
    bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(c->d_status, (long long)limit_cycles, gave_up);
    return launch_status(c, "bounded_wait_selftest_kernel");
}

extern "C" uint64_t fxb_launch_count(fxb_handle_t h) {
    return h ? reinterpret_cast<Context*>(h)->launches : 0;
}

extern "C" const char* fxb_status_string(int status) {
    switch (status) {
        case FXB_OK: return "ok";
        case FXB_ERR_INVALID_ARGUMENT: return "invalid argument";
        case FXB_ERR_UNSUPPORTED: return "unsupported";
        case FXB_ERR_LAUNCH_FAILED: return "kernel launch failed";
        case FXB_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait ran out";
        case FXB_ERR_CUDA: return "CUDA runtime error";
        case FXB_ERR_WORKSPACE: return "workspace too small";
        default: return "unknown status";
    }
}

extern "C" int fxb_create(int device, fxb_handle_t* out) {
    if (out == nullptr) return fail(nullptr, FXB_ERR_INVALID_ARGUMENT, "fxb_create: out is null");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        return fail(nullptr, FXB_ERR_CUDA, std::string("fxb_create: no CUDA device available: ") + cudaGetErrorString(e));
    if (device < 0 || device >= count)
        return fail(nullptr, FXB_ERR_INVALID_ARGUMENT, "fxb_create: device id out of range");
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) return fail(nullptr, FXB_ERR_CUDA, std::string("fxb_create: ") + cudaGetErrorString(e));
    if (prop.major != 10)
        return fail(nullptr, FXB_ERR_UNSUPPORTED,
                    "fxb_create: this library is built for sm_100a (B200) only; device is sm_" +
                        std::to_string(prop.major) + std::to_string(prop.minor));
    int prev = 0;
    cudaGetDevice(&prev);
    e = cudaSetDevice(device);
    if (e != cudaSuccess) return fail(nullptr, FXB_ERR_CUDA, std::string("fxb_create: ") + cudaGetErrorString(e));
    Context* c = new Context();
    c->device = device;
    c->sm_count = prop.multiProcessorCount;
    e = cudaMalloc(reinterpret_cast<void**>(&c->d_status), sizeof(DeviceStatus) + 8192);
    if (e == cudaSuccess) e = cudaMemset(c->d_status, 0, sizeof(DeviceStatus) + 8192);
    c->d_scratch = reinterpret_cast<char*>(c->d_status) + sizeof(DeviceStatus);
    // the static scratch array's device address, looked up while this device is current
    const int rs = e == cudaSuccess ? resolve_static_scratch(c) : FXB_OK;
    cudaSetDevice(prev);
    if (e != cudaSuccess) {
        delete c;
        return fail(nullptr, FXB_ERR_CUDA, std::string("fxb_create: status block: ") + cudaGetErrorString(e));
    }
    if (rs != FXB_OK) {
        const std::string msg = c->last_error;
        cudaFree(c->d_status);
        delete c;
        return fail(nullptr, rs, "fxb_create: " + msg);
    }
    *out = reinterpret_cast<fxb_handle_t>(c);
    return FXB_OK;
}

extern "C" int fxb_destroy(fxb_handle_t h) {
    if (h == nullptr) return FXB_OK;
    Context* c = reinterpret_cast<Context*>(h);
    if (c->d_status) cudaFree(c->d_status);
    delete c;
    return FXB_OK;
}

extern "C" const char* fxb_last_error(fxb_handle_t h) {
    if (h == nullptr) return g_tls_error.c_str();
    return reinterpret_cast<Context*>(h)->last_error.c_str();
}

extern "C" int fxb_set_math_mode(fxb_handle_t h, int mode) {
    if (h == nullptr) return fail(nullptr, FXB_ERR_INVALID_ARGUMENT, "null ferrox_b200 handle");
    Context* c = reinterpret_cast<Context*>(h);
    if (mode != FXB_MATH_3XTF32 && mode != FXB_MATH_TF32) return fail(c, FXB_ERR_INVALID_ARGUMENT, "unknown math mode");
    c->math_mode = mode;
    return FXB_OK;
}

extern "C" int fxb_set_operand_path(fxb_handle_t h, int path) {
    if (h == nullptr) return fail(nullptr, FXB_ERR_INVALID_ARGUMENT, "null ferrox_b200 handle");
    Context* c = reinterpret_cast<Context*>(h);
    if (path != FXB_PATH_AUTO && path != FXB_PATH_GATHER && path != FXB_PATH_CP_ASYNC)
        return fail(c, FXB_ERR_INVALID_ARGUMENT, "unknown operand path");
    c->operand_path = path;
    return FXB_OK;
}

extern "C" int fxb_set_accumulate_stages(fxb_handle_t h, int stages) {
    if (h == nullptr) return fail(nullptr, FXB_ERR_INVALID_ARGUMENT, "null ferrox_b200 handle");
    Context* c = reinterpret_cast<Context*>(h);
    if (stages != 1 && stages != 2 && stages != 4) return fail(c, FXB_ERR_INVALID_ARGUMENT, "accumulate stages must be 1, 2 or 4");
    c->drain_group = stages;
    return FXB_OK;
}

extern "C" int fxb_set_sigmoid_grad_mode(fxb_handle_t h, int math_mode) {
    if (h == nullptr) return fail(nullptr, FXB_ERR_INVALID_ARGUMENT, "null ferrox_b200 handle");
    reinterpret_cast<Context*>(h)->sigmoid_grad_math = math_mode ? 1 : 0;
    return FXB_OK;
}

extern "C" int fxb_check_device_status(fxb_handle_t h, fxb_stream_t stream) {
    if (h == nullptr) return fail(nullptr, FXB_ERR_INVALID_ARGUMENT, "null ferrox_b200 handle");
    Context* c = reinterpret_cast<Context*>(h);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    DeviceStatus hs;
    FXB_CUDA_OK(c, cudaMemcpyAsync(&hs, c->d_status, sizeof(hs), cudaMemcpyDeviceToHost, st));
    FXB_CUDA_OK(c, cudaStreamSynchronize(st));
    if (hs.code != 0) {
        cudaMemsetAsync(c->d_status, 0, sizeof(DeviceStatus), st);
        cudaStreamSynchronize(st);
        return fail(c, FXB_ERR_DEVICE_TIMEOUT,
                    "device-side wait ran out (tag " + std::to_string(hs.where) + ", block " +
                        std::to_string(hs.block_x) + "," + std::to_string(hs.block_y) + "," +
                        std::to_string(hs.block_z) + ")");
    }
    return FXB_OK;
}

// Run-time compilation and launch of the element-wise / reduction kernels that the Python
// float_ew compiler generates as CUDA-C source. Stands in for pycuda.compiler.SourceModule +
// Function.prepare + prepared_async_call (nervanagpu/float_ew.py:1030-1035,1314).
// Source -> NVRTC (sm_100a cubin) -> driver module -> cuLaunchKernel.
#include <nvrtc.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/nervana_b200.h"
#include "host.h"

namespace ngb {
namespace {

struct DriverApi {
  CUresult (*moduleLoadData)(CUmodule*, const void*) = nullptr;
  CUresult (*moduleUnload)(CUmodule) = nullptr;
  CUresult (*moduleGetFunction)(CUfunction*, CUmodule, const char*) = nullptr;
  CUresult (*launchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream,
                           void**, void**) = nullptr;
  CUresult (*funcSetAttribute)(CUfunction, CUfunction_attribute, int) = nullptr;
  bool ok = false;
};

template <typename F>
bool load_sym(const char* name, F& fn) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPointByVersion(name, &p, 12000, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return false;
  fn = reinterpret_cast<F>(p);
  return true;
}

DriverApi& driver() {
  static DriverApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    api.ok = load_sym("cuModuleLoadData", api.moduleLoadData) && load_sym("cuModuleUnload", api.moduleUnload) &&
             load_sym("cuModuleGetFunction", api.moduleGetFunction) && load_sym("cuLaunchKernel", api.launchKernel) &&
             load_sym("cuFuncSetAttribute", api.funcSetAttribute);
  });
  return api;
}

struct EwKernel {
  CUmodule mod;
  CUfunction fn;
};

std::string g_log;
std::mutex g_log_mutex;

}  // namespace
}  // namespace ngb

using namespace ngb;

extern "C" {

const char* ng_ew_compile_log(void) {
  std::lock_guard<std::mutex> lock(g_log_mutex);
  return g_log.c_str();
}

// NVRTC front half: source -> sm_100a cubin. Needs no device.
static int compile_to_cubin(const char* source, int fast_math, std::vector<char>& cubin) {
  nvrtcProgram prog;
  nvrtcResult r = nvrtcCreateProgram(&prog, source, "ew_kernel.cu", 0, nullptr, nullptr);
  if (r != NVRTC_SUCCESS) return fail(NG_ERR_NVRTC, "nvrtcCreateProgram: %s", nvrtcGetErrorString(r));
  const char* cuda_home = getenv("CUDA_HOME");
  std::string inc = std::string("--include-path=") + (cuda_home ? cuda_home : "/usr/local/cuda") + "/include";
  std::vector<const char*> opts = {"--gpu-architecture=sm_100a", "--std=c++17", "-default-device", inc.c_str()};
  // Without fast math every operation rounds once, in source order, like the numpy fp32 oracle:
  // no contraction of a*b+c into an fma.
  if (fast_math) opts.push_back("--use_fast_math");
  else opts.push_back("--fmad=false");
  r = nvrtcCompileProgram(prog, static_cast<int>(opts.size()), opts.data());
  size_t log_size = 0;
  nvrtcGetProgramLogSize(prog, &log_size);
  {
    std::lock_guard<std::mutex> lock(g_log_mutex);
    g_log.assign(log_size ? log_size : 1, '\0');
    if (log_size) nvrtcGetProgramLog(prog, &g_log[0]);
  }
  if (r != NVRTC_SUCCESS) {
    nvrtcDestroyProgram(&prog);
    return fail(NG_ERR_NVRTC, "nvrtcCompileProgram failed: %s (see ng_ew_compile_log)", nvrtcGetErrorString(r));
  }
  size_t cubin_size = 0;
  r = nvrtcGetCUBINSize(prog, &cubin_size);
  if (r != NVRTC_SUCCESS || cubin_size == 0) {
    nvrtcDestroyProgram(&prog);
    return fail(NG_ERR_NVRTC, "nvrtcGetCUBINSize: %s", nvrtcGetErrorString(r));
  }
  cubin.resize(cubin_size);
  nvrtcGetCUBIN(prog, cubin.data());
  nvrtcDestroyProgram(&prog);
  return NG_OK;
}

int ng_ew_compile_only(const char* source, int fast_math) {
  if (!source) return fail(NG_ERR_INVALID_ARG, "null argument");
  std::vector<char> cubin;
  return compile_to_cubin(source, fast_math, cubin);
}

int ng_ew_compile(const char* source, const char* kernel_name, int fast_math, void** handle) {
  if (!source || !kernel_name || !handle) return fail(NG_ERR_INVALID_ARG, "null argument");
  DeviceCtx* c = current_ctx();
  if (!c) return NG_ERR_CUDA;
  DriverApi& api = driver();
  if (!api.ok) return fail(NG_ERR_CUDA, "driver module entry points not available");
  std::vector<char> cubin;
  int crc = compile_to_cubin(source, fast_math, cubin);
  if (crc != NG_OK) return crc;

  EwKernel* k = new EwKernel();
  CUresult cr = api.moduleLoadData(&k->mod, cubin.data());
  if (cr != CUDA_SUCCESS) {
    delete k;
    return fail(NG_ERR_CUDA, "cuModuleLoadData failed (%d)", static_cast<int>(cr));
  }
  cr = api.moduleGetFunction(&k->fn, k->mod, kernel_name);
  if (cr != CUDA_SUCCESS) {
    api.moduleUnload(k->mod);
    delete k;
    return fail(NG_ERR_CUDA, "kernel '%s' not found in compiled module (%d)", kernel_name, static_cast<int>(cr));
  }
  *handle = k;
  return NG_OK;
}

int ng_ew_launch(void* handle, unsigned gx, unsigned gy, unsigned gz, unsigned bx, unsigned by, unsigned bz,
                 unsigned shared_bytes, void** args, void* stream) {
  if (!handle) return fail(NG_ERR_INVALID_ARG, "null kernel handle");
  if (gx == 0 || gy == 0 || gz == 0 || bx == 0 || by == 0 || bz == 0) return NG_OK;  // empty launch
  EwKernel* k = static_cast<EwKernel*>(handle);
  DriverApi& api = driver();
  CUresult cr = api.launchKernel(k->fn, gx, gy, gz, bx, by, bz, shared_bytes, static_cast<CUstream>(stream), args,
                                 nullptr);
  if (cr != CUDA_SUCCESS) return fail(NG_ERR_CUDA, "cuLaunchKernel failed (%d)", static_cast<int>(cr));
  count_launch();
  return NG_OK;
}

int ng_ew_release(void* handle) {
  if (!handle) return NG_OK;
  EwKernel* k = static_cast<EwKernel*>(handle);
  driver().moduleUnload(k->mod);
  delete k;
  return NG_OK;
}

}  // extern "C"

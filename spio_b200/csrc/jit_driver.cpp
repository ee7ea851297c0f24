// Just-in-time path of libspio_b200: NVRTC compilation to sm_100a cubins and module load /
// kernel launch through the CUDA driver API.
//
// Native counterpart of the reference's two binding layers:
//   spio/cuda/nvrtc_ctypes.py:152-217  (NVRTC Program: create, compile, log, cubin)
//   spio/cuda/driver.pyx:126-273       (Module.load_data, get_function, Function.launch)
// Differences: launches go to a caller-supplied stream (the reference uses the NULL stream,
// driver.pyx:200-208), arguments are passed as the driver's void** array, so by-value structs
// such as 128-byte tensor maps work, and neither libnvrtc nor libcuda is a link-time
// dependency (dlopen / cudaGetDriverEntryPoint).
#include <cuda.h>
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cstdio>
#include <cstdlib>
#include <atomic>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/spio_b200.h"

namespace spio_b200 {
int jit_fail(const std::string& msg);  // sets the thread's last-error string, returns 1
}
using spio_b200::jit_fail;

namespace {

// ---------------------------------------------------------------- NVRTC (loaded on demand)
typedef int nvrtcResult;
typedef struct _nvrtcProgram* nvrtcProgram;
struct Nvrtc {
  void* handle = nullptr;
  nvrtcResult (*CreateProgram)(nvrtcProgram*, const char*, const char*, int, const char* const*,
                               const char* const*) = nullptr;
  nvrtcResult (*CompileProgram)(nvrtcProgram, int, const char* const*) = nullptr;
  nvrtcResult (*DestroyProgram)(nvrtcProgram*) = nullptr;
  nvrtcResult (*GetProgramLogSize)(nvrtcProgram, size_t*) = nullptr;
  nvrtcResult (*GetProgramLog)(nvrtcProgram, char*) = nullptr;
  nvrtcResult (*GetCUBINSize)(nvrtcProgram, size_t*) = nullptr;
  nvrtcResult (*GetCUBIN)(nvrtcProgram, char*) = nullptr;
  const char* (*GetErrorString)(nvrtcResult) = nullptr;
  nvrtcResult (*Version)(int*, int*) = nullptr;
};
Nvrtc g_nvrtc;
std::string g_nvrtc_path;
std::mutex g_jit_mutex;

template <class F>
bool sym(void* h, const char* name, F& fn) {
  fn = reinterpret_cast<F>(dlsym(h, name));
  return fn != nullptr;
}

int load_nvrtc() {
  std::lock_guard<std::mutex> lock(g_jit_mutex);
  if (g_nvrtc.handle) return 0;
  std::vector<std::string> names;
  if (!g_nvrtc_path.empty()) names.push_back(g_nvrtc_path);
  if (const char* env = getenv("SPIO_NVRTC_PATH")) names.push_back(env);
  names.push_back("libnvrtc.so.12");
  names.push_back("libnvrtc.so");
  names.push_back("/usr/local/cuda/lib64/libnvrtc.so");
  void* h = nullptr;
  for (const std::string& n : names) {
    h = dlopen(n.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (h) break;
  }
  if (!h) return jit_fail("NVRTC library not found (set SPIO_NVRTC_PATH or call spio_jit_set_nvrtc_path)");
  Nvrtc n;
  n.handle = h;
  const bool ok = sym(h, "nvrtcCreateProgram", n.CreateProgram) && sym(h, "nvrtcCompileProgram", n.CompileProgram) &&
                  sym(h, "nvrtcDestroyProgram", n.DestroyProgram) &&
                  sym(h, "nvrtcGetProgramLogSize", n.GetProgramLogSize) &&
                  sym(h, "nvrtcGetProgramLog", n.GetProgramLog) && sym(h, "nvrtcGetCUBINSize", n.GetCUBINSize) &&
                  sym(h, "nvrtcGetCUBIN", n.GetCUBIN) && sym(h, "nvrtcGetErrorString", n.GetErrorString) &&
                  sym(h, "nvrtcVersion", n.Version);
  if (!ok) return jit_fail("NVRTC library lacks a required symbol");
  g_nvrtc = n;
  return 0;
}

// ---------------------------------------------------------------- driver API (entry points)
struct Driver {
  bool ready = false;
  CUresult (*ModuleLoadData)(CUmodule*, const void*) = nullptr;
  CUresult (*ModuleUnload)(CUmodule) = nullptr;
  CUresult (*ModuleGetFunction)(CUfunction*, CUmodule, const char*) = nullptr;
  CUresult (*FuncSetAttribute)(CUfunction, CUfunction_attribute, int) = nullptr;
  CUresult (*FuncGetAttribute)(int*, CUfunction_attribute, CUfunction) = nullptr;
  CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned,
                           CUstream, void**, void**) = nullptr;
  CUresult (*LaunchKernelEx)(const CUlaunchConfig*, CUfunction, void**, void**) = nullptr;
  CUresult (*GetErrorString)(CUresult, const char**) = nullptr;
};
Driver g_drv;

template <class F>
bool entry(const char* name, F& fn) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || p == nullptr ||
      q != cudaDriverEntryPointSuccess)
    return false;
  fn = reinterpret_cast<F>(p);
  return true;
}

std::atomic<bool> g_drv_ready{false};

int load_driver() {
  if (g_drv_ready.load(std::memory_order_acquire)) return 0;  // the usual case takes no lock
  std::lock_guard<std::mutex> lock(g_jit_mutex);
  if (g_drv.ready) return 0;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaSetDevice(dev);  // binds the primary context to this thread
  if (e != cudaSuccess) return jit_fail(std::string("CUDA error: ") + cudaGetErrorString(e));
  Driver d;
  const bool ok = entry("cuModuleLoadData", d.ModuleLoadData) && entry("cuModuleUnload", d.ModuleUnload) &&
                  entry("cuModuleGetFunction", d.ModuleGetFunction) &&
                  entry("cuFuncSetAttribute", d.FuncSetAttribute) &&
                  entry("cuFuncGetAttribute", d.FuncGetAttribute) && entry("cuLaunchKernel", d.LaunchKernel) &&
                  entry("cuLaunchKernelEx", d.LaunchKernelEx) && entry("cuGetErrorString", d.GetErrorString);
  if (!ok) return jit_fail("CUDA error: a driver entry point is not available");
  d.ready = true;
  g_drv = d;
  g_drv_ready.store(true, std::memory_order_release);
  return 0;
}

int drv_fail(const char* what, CUresult r) {
  const char* msg = nullptr;
  if (g_drv.GetErrorString) g_drv.GetErrorString(r, &msg);
  return jit_fail(std::string("CUDA error: ") + (msg ? msg : "unknown") + " (" + what + ")");
}

int bind_context() {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaSetDevice(dev);
  if (e != cudaSuccess) return jit_fail(std::string("CUDA error: ") + cudaGetErrorString(e));
  return 0;
}

}  // namespace

namespace spio_b200 {

// cuLaunchKernelEx on the caller's stream, optionally with the programmatic-stream-serialization
// attribute the kernels built into the library are launched with, so that a just-in-time kernel
// takes part in a chain of dependent launches like any other (the reference launches with plain
// cuLaunchKernel on the NULL stream, spio/cuda/driver.pyx:200-208).
int jit_launch(void* function, int grid, int block, int smem_bytes, cudaStream_t stream, void** args,
               bool programmatic) {
  if (function == nullptr) return jit_fail("NULL function");
  if (grid <= 0 || block <= 0 || block > 1024) return jit_fail("bad launch dimensions");
  if (load_driver()) return 1;
  CUlaunchConfig cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.gridDimX = (unsigned)grid, cfg.gridDimY = 1, cfg.gridDimZ = 1;
  cfg.blockDimX = (unsigned)block, cfg.blockDimY = 1, cfg.blockDimZ = 1;
  cfg.sharedMemBytes = (unsigned)smem_bytes;
  cfg.hStream = static_cast<CUstream>(stream);
  CUlaunchAttribute attr[1];
  memset(attr, 0, sizeof attr);
  attr[0].id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
  attr[0].value.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = programmatic ? 1 : 0;
  const CUresult r = g_drv.LaunchKernelEx(&cfg, static_cast<CUfunction>(function), args, nullptr);
  return r == CUDA_SUCCESS ? 0 : drv_fail("cuLaunchKernelEx", r);
}

}  // namespace spio_b200

extern "C" {

int spio_jit_set_nvrtc_path(const char* path) {
  std::lock_guard<std::mutex> lock(g_jit_mutex);
  g_nvrtc_path = path ? path : "";
  return 0;
}

int spio_jit_nvrtc_version(int* major, int* minor) {
  if (load_nvrtc()) return 1;
  return g_nvrtc.Version(major, minor) == 0 ? 0 : jit_fail("nvrtcVersion failed");
}

int spio_jit_compile(const char* source, const char* file_name, const char* const* options, int n_options,
                     const char* const* header_names, const char* const* header_sources, int n_headers,
                     void** cubin, size_t* cubin_size, char** log) {
  if (source == nullptr || cubin == nullptr || cubin_size == nullptr) return jit_fail("NULL argument");
  *cubin = nullptr;
  *cubin_size = 0;
  if (log) *log = nullptr;
  if (load_nvrtc()) return 1;
  nvrtcProgram prog = nullptr;
  nvrtcResult r = g_nvrtc.CreateProgram(&prog, source, file_name ? file_name : "kernel.cu", n_headers,
                                        header_sources, header_names);
  if (r != 0) return jit_fail(std::string("nvrtcCreateProgram: ") + g_nvrtc.GetErrorString(r));
  r = g_nvrtc.CompileProgram(prog, n_options, options);
  size_t log_size = 0;
  g_nvrtc.GetProgramLogSize(prog, &log_size);
  std::string text(log_size > 0 ? log_size : 1, '\0');
  if (log_size > 1) g_nvrtc.GetProgramLog(prog, &text[0]);
  if (log) {
    *log = static_cast<char*>(malloc(text.size() + 1));
    if (*log) memcpy(*log, text.c_str(), text.size() + 1);
  }
  if (r != 0) {
    g_nvrtc.DestroyProgram(&prog);
    return jit_fail("Compilation error log: " + text);
  }
  size_t size = 0;
  r = g_nvrtc.GetCUBINSize(prog, &size);
  if (r != 0 || size == 0) {
    g_nvrtc.DestroyProgram(&prog);
    return jit_fail("nvrtcGetCUBINSize failed (was -arch=sm_XY given?)");
  }
  void* buf = malloc(size);
  if (!buf) {
    g_nvrtc.DestroyProgram(&prog);
    return jit_fail("out of host memory");
  }
  r = g_nvrtc.GetCUBIN(prog, static_cast<char*>(buf));
  g_nvrtc.DestroyProgram(&prog);
  if (r != 0) {
    free(buf);
    return jit_fail("nvrtcGetCUBIN failed");
  }
  *cubin = buf;
  *cubin_size = size;
  return 0;
}

void spio_jit_free(void* p) { free(p); }

int spio_module_load(const void* cubin, void** module) {
  if (cubin == nullptr || module == nullptr) return jit_fail("NULL argument");
  if (load_driver() || bind_context()) return 1;
  CUmodule m = nullptr;
  const CUresult r = g_drv.ModuleLoadData(&m, cubin);
  if (r != CUDA_SUCCESS) return drv_fail("cuModuleLoadData", r);
  *module = m;
  return 0;
}

int spio_module_unload(void* module) {
  if (module == nullptr) return 0;
  if (load_driver() || bind_context()) return 1;
  const CUresult r = g_drv.ModuleUnload(static_cast<CUmodule>(module));
  return r == CUDA_SUCCESS ? 0 : drv_fail("cuModuleUnload", r);
}

int spio_module_get_function(void* module, const char* name, void** function) {
  if (module == nullptr || name == nullptr || function == nullptr) return jit_fail("NULL argument");
  if (load_driver()) return 1;
  CUfunction f = nullptr;
  const CUresult r = g_drv.ModuleGetFunction(&f, static_cast<CUmodule>(module), name);
  if (r != CUDA_SUCCESS) return drv_fail("cuModuleGetFunction", r);
  *function = f;
  return 0;
}

int spio_function_set_max_dynamic_smem(void* function, int bytes) {
  if (load_driver()) return 1;
  const CUresult r = g_drv.FuncSetAttribute(static_cast<CUfunction>(function),
                                            CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, bytes);
  return r == CUDA_SUCCESS ? 0 : drv_fail("cuFuncSetAttribute", r);
}

int spio_function_get_attribute(void* function, int which, int* value) {
  if (value == nullptr) return jit_fail("NULL argument");
  if (load_driver()) return 1;
  CUfunction_attribute a;
  switch (which) {
    case 0: a = CU_FUNC_ATTRIBUTE_NUM_REGS; break;
    case 1: a = CU_FUNC_ATTRIBUTE_LOCAL_SIZE_BYTES; break;
    case 2: a = CU_FUNC_ATTRIBUTE_SHARED_SIZE_BYTES; break;
    case 3: a = CU_FUNC_ATTRIBUTE_MAX_THREADS_PER_BLOCK; break;
    default: return jit_fail("unknown function attribute");
  }
  const CUresult r = g_drv.FuncGetAttribute(value, a, static_cast<CUfunction>(function));
  return r == CUDA_SUCCESS ? 0 : drv_fail("cuFuncGetAttribute", r);
}

int spio_function_launch(void* function, int grid, int block, int smem_bytes, void* stream, void** args) {
  if (function == nullptr) return jit_fail("NULL function");
  if (grid <= 0 || block <= 0 || block > 1024) return jit_fail("bad launch dimensions");
  if (load_driver() || bind_context()) return 1;
  const CUresult r = g_drv.LaunchKernel(static_cast<CUfunction>(function), (unsigned)grid, 1, 1, (unsigned)block,
                                        1, 1, (unsigned)smem_bytes, static_cast<CUstream>(stream), args, nullptr);
  return r == CUDA_SUCCESS ? 0 : drv_fail("cuLaunchKernel", r);
}

int spio_function_launch_ex(void* function, int grid, int block, int smem_bytes, void* stream, void** args,
                            int flags) {
  if (bind_context()) return 1;
  return spio_b200::jit_launch(function, grid, block, smem_bytes, static_cast<cudaStream_t>(stream), args,
                               (flags & SPIO_LAUNCH_PROGRAMMATIC) != 0);
}

}  // extern "C"

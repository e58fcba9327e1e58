// Runtime specialisation of edge programs: CUDA source generated for ONE staged edge expression
// (straight-line code instead of the interpreter's instruction loop) is compiled for sm_100a with
// NVRTC and launched through the driver's module interface.
//
// This is the role the reference gives its provider pipeline -- a captured edge UDF becomes
// generated kernel code that a runtime compiler turns into a binary, cached per specialisation
// (python/tiga/codegen/ttir.py:103-121 `prepare_ttir_*`, python/tiga/interop/torch/message_passing.py:
// 2579-2815 `_execute_generic_csr` of walkerchi/TIGA-lang, whose compiler is Triton).  Here the source
// is CUDA C++ written by tiga/edge_jit.py from the same kernels as csrc/tgb_edge_program.cu.
//
// NVRTC is opened at run time (dlopen), so the library has no link-time dependency on it; building
// a module needs no GPU (the compile check runs anywhere), loading and launching do.
#include <dlfcn.h>

#include <cuda.h>

#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "tgb_common.cuh"

namespace tgb {
namespace {

struct Nvrtc {
  void *handle = nullptr;
  int (*create)(void **, const char *, const char *, int, const char *const *, const char *const *) = nullptr;
  int (*compile)(void *, int, const char *const *) = nullptr;
  int (*log_size)(void *, size_t *) = nullptr;
  int (*get_log)(void *, char *) = nullptr;
  int (*cubin_size)(void *, size_t *) = nullptr;
  int (*get_cubin)(void *, char *) = nullptr;
  int (*destroy)(void **) = nullptr;
  const char *(*error_string)(int) = nullptr;
};

const Nvrtc *nvrtc() {
  static Nvrtc api;
  static std::once_flag once;
  std::call_once(once, [] {
    const char *names[] = {"libnvrtc.so.12", "/usr/local/cuda/lib64/libnvrtc.so.12", "libnvrtc.so"};
    for (const char *name : names) {
      api.handle = dlopen(name, RTLD_NOW | RTLD_LOCAL);
      if (api.handle) break;
    }
    if (!api.handle) return;
    auto load = [&](const char *symbol) { return dlsym(api.handle, symbol); };
    api.create = reinterpret_cast<decltype(api.create)>(load("nvrtcCreateProgram"));
    api.compile = reinterpret_cast<decltype(api.compile)>(load("nvrtcCompileProgram"));
    api.log_size = reinterpret_cast<decltype(api.log_size)>(load("nvrtcGetProgramLogSize"));
    api.get_log = reinterpret_cast<decltype(api.get_log)>(load("nvrtcGetProgramLog"));
    api.cubin_size = reinterpret_cast<decltype(api.cubin_size)>(load("nvrtcGetCUBINSize"));
    api.get_cubin = reinterpret_cast<decltype(api.get_cubin)>(load("nvrtcGetCUBIN"));
    api.destroy = reinterpret_cast<decltype(api.destroy)>(load("nvrtcDestroyProgram"));
    api.error_string = reinterpret_cast<decltype(api.error_string)>(load("nvrtcGetErrorString"));
    if (!api.create || !api.compile || !api.log_size || !api.get_log || !api.cubin_size || !api.get_cubin ||
        !api.destroy)
      api.handle = nullptr;
  });
  return api.handle ? &api : nullptr;
}

struct Driver {
  CUresult (*module_load)(CUmodule *, const void *) = nullptr;
  CUresult (*module_function)(CUfunction *, CUmodule, const char *) = nullptr;
  CUresult (*module_unload)(CUmodule) = nullptr;
  CUresult (*launch)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream,
                     void **, void **) = nullptr;
  CUresult (*function_attribute)(int *, CUfunction_attribute, CUfunction) = nullptr;
  CUresult (*current_context)(CUcontext *) = nullptr;
  bool ok = false;
};

const Driver *driver() {
  static Driver api;
  static std::once_flag once;
  std::call_once(once, [] {
    auto load = [](const char *symbol) -> void * {
      void *fn = nullptr;
      cudaDriverEntryPointQueryResult query;
      if (cudaGetDriverEntryPoint(symbol, &fn, cudaEnableDefault, &query) != cudaSuccess ||
          query != cudaDriverEntryPointSuccess)
        return nullptr;
      return fn;
    };
    api.module_load = reinterpret_cast<decltype(api.module_load)>(load("cuModuleLoadData"));
    api.module_function = reinterpret_cast<decltype(api.module_function)>(load("cuModuleGetFunction"));
    api.module_unload = reinterpret_cast<decltype(api.module_unload)>(load("cuModuleUnload"));
    api.launch = reinterpret_cast<decltype(api.launch)>(load("cuLaunchKernel"));
    api.function_attribute = reinterpret_cast<decltype(api.function_attribute)>(load("cuFuncGetAttribute"));
    api.current_context = reinterpret_cast<decltype(api.current_context)>(load("cuCtxGetCurrent"));
    api.ok = api.module_load && api.module_function && api.module_unload && api.launch && api.function_attribute &&
             api.current_context;
  });
  return api.ok ? &api : nullptr;
}

constexpr int kMaxDevices = 64;

}  // namespace
}  // namespace tgb

// One compiled source: the binary image, and per device the loaded module with its kernels by name.
struct tgb_jit_module {
  std::vector<char> image;
  std::mutex lock;
  CUmodule loaded[tgb::kMaxDevices] = {};
  std::map<std::string, CUfunction> kernels[tgb::kMaxDevices];
};

using namespace tgb;

extern "C" int32_t tgb_jit_build(const char *source, tgb_jit_module **module, char *log, int64_t log_capacity) {
  if (!source || !module) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null argument");
  if (log && log_capacity > 0) log[0] = '\0';
  const Nvrtc *rtc = nvrtc();
  if (!rtc) TGB_FAIL(TGB_STATUS_UNSUPPORTED, "the NVRTC library (libnvrtc.so.12) could not be opened");
  void *program = nullptr;
  int rc = rtc->create(&program, source, "tiga_edge_program.cu", 0, nullptr, nullptr);
  if (rc != 0) TGB_FAIL(TGB_STATUS_INTERNAL, "nvrtcCreateProgram failed (%d)", rc);
  const char *options[] = {"--gpu-architecture=sm_100a", "--std=c++17", "-lineinfo"};
  rc = rtc->compile(program, 3, options);
  size_t size = 0;
  if (log && log_capacity > 0 && rtc->log_size(program, &size) == 0 && size > 1) {
    std::vector<char> text(size);
    rtc->get_log(program, text.data());
    const size_t n = size - 1 < (size_t)log_capacity - 1 ? size - 1 : (size_t)log_capacity - 1;
    memcpy(log, text.data(), n);
    log[n] = '\0';
  }
  if (rc != 0) {
    rtc->destroy(&program);
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "the generated source did not compile (nvrtc %d: %s)", rc,
             rtc->error_string ? rtc->error_string(rc) : "?");
  }
  auto *built = new tgb_jit_module();
  if (rtc->cubin_size(program, &size) != 0 || size == 0) {
    rtc->destroy(&program);
    delete built;
    TGB_FAIL(TGB_STATUS_INTERNAL, "nvrtc produced no binary");
  }
  built->image.resize(size);
  rtc->get_cubin(program, built->image.data());
  rtc->destroy(&program);
  *module = built;
  return TGB_STATUS_OK;
}

extern "C" int32_t tgb_jit_image_bytes(const tgb_jit_module *module, int64_t *bytes) {
  if (!module || !bytes) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null argument");
  *bytes = (int64_t)module->image.size();
  return TGB_STATUS_OK;
}

extern "C" int32_t tgb_jit_launch(tgb_jit_module *module, const char *kernel, uint32_t grid, uint32_t block,
                                  const void *arguments, uint64_t stream) {
  if (!module || !kernel || !arguments) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null argument");
  if (grid == 0) return TGB_STATUS_OK;
  const Driver *api = driver();
  if (!api) TGB_FAIL(TGB_STATUS_INTERNAL, "the driver's module interface is not available");
  int device = 0;
  TGB_CUDA(cudaGetDevice(&device));
  if (device < 0 || device >= kMaxDevices) TGB_FAIL(TGB_STATUS_UNSUPPORTED, "device ordinal out of range");
  // A thread that has made no runtime call yet (an autograd worker) has no context bound; the
  // no-op free binds the primary one.  Threads that have a context skip it, which also keeps the
  // launch legal while a stream is being captured into a CUDA graph.
  CUcontext current = nullptr;
  if (api->current_context(&current) != CUDA_SUCCESS || current == nullptr) TGB_CUDA(cudaFree(nullptr));
  CUfunction function = nullptr;
  {
    std::lock_guard<std::mutex> guard(module->lock);
    if (!module->loaded[device]) {
      const CUresult rc = api->module_load(&module->loaded[device], module->image.data());
      if (rc != CUDA_SUCCESS) {
        module->loaded[device] = nullptr;
        TGB_FAIL(TGB_STATUS_INTERNAL, "cuModuleLoadData failed (%d)", (int)rc);
      }
    }
    auto found = module->kernels[device].find(kernel);
    if (found == module->kernels[device].end()) {
      const CUresult rc = api->module_function(&function, module->loaded[device], kernel);
      if (rc != CUDA_SUCCESS) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "kernel %s is not in the module (%d)", kernel, (int)rc);
      module->kernels[device][kernel] = function;
    } else {
      function = found->second;
    }
  }
  if (block == 0) {     // the block size the kernel was compiled for (its __launch_bounds__)
    int limit = 0;
    const CUresult rc = api->function_attribute(&limit, CU_FUNC_ATTRIBUTE_MAX_THREADS_PER_BLOCK, function);
    if (rc != CUDA_SUCCESS || limit < 32) TGB_FAIL(TGB_STATUS_INTERNAL, "cuFuncGetAttribute(%s) failed (%d)", kernel, (int)rc);
    block = (uint32_t)limit;
  }
  // every generated kernel takes ONE by-value argument (its argument block)
  void *params[1] = {const_cast<void *>(arguments)};
  const CUresult rc = api->launch(function, grid, 1, 1, block, 1, 1, 0, reinterpret_cast<CUstream>(stream), params,
                                  nullptr);
  if (rc != CUDA_SUCCESS) TGB_FAIL(TGB_STATUS_INTERNAL, "cuLaunchKernel(%s) failed (%d)", kernel, (int)rc);
  g_launches.fetch_add(1);
  return TGB_STATUS_OK;
}

extern "C" void tgb_jit_destroy(tgb_jit_module *module) {
  if (!module) return;
  const Driver *api = driver();
  for (int device = 0; device < kMaxDevices; ++device)
    if (module->loaded[device] && api) {
      int current = 0;
      if (cudaGetDevice(&current) == cudaSuccess && cudaSetDevice(device) == cudaSuccess) {
        api->module_unload(module->loaded[device]);
        cudaSetDevice(current);
      }
    }
  delete module;
}

// Name-keyed kernel registry, kept for API and test parity with the reference
// (infini_train/include/dispatcher.h:13-62, test/kernels/test_dispatcher.cc).  The hot path of
// this framework calls its sm_100a kernels directly; the registry maps {device type, name} to a
// type-erased function pointer so that user code written against
//   Dispatcher::Instance().GetKernel({device, "LinearForward"}).Call<Ret>(args...)
// and REGISTER_KERNEL(device, name, fn) keeps working.
#pragma once
#include <map>
#include <stdexcept>
#include <string>
#include <utility>

#include "core/framework/tensor.h"

namespace infini_train {

class KernelFunction {
 public:
  KernelFunction() = default;
  template <typename FuncT>
  explicit KernelFunction(FuncT&& func) : func_ptr_(reinterpret_cast<void*>(func)) {}

  // The caller states the return type; argument types are taken from the call site and must match
  // the registered function's signature exactly (as in the reference).
  template <typename RetT, class... ArgsT>
  RetT Call(ArgsT... args) const {
    using FuncT = RetT (*)(ArgsT...);
    auto fn = reinterpret_cast<FuncT>(func_ptr_);
    return fn(args...);
  }

 private:
  void* func_ptr_ = nullptr;
};

class Dispatcher {
 public:
  using KeyT = std::pair<DeviceType, std::string>;

  static Dispatcher& Instance() {
    static Dispatcher instance;
    return instance;
  }

  const KernelFunction& GetKernel(const KeyT& key) const {
    auto it = key_to_kernel_map_.find(key);
    if (it == key_to_kernel_map_.end())
      throw std::runtime_error("Kernel not found: " + key.second + " on device " + std::to_string(static_cast<int>(key.first)));
    return it->second;
  }
  bool HasKernel(const KeyT& key) const { return key_to_kernel_map_.count(key) != 0; }

  template <typename FuncT>
  void Register(const KeyT& key, FuncT&& kernel) {
    if (key_to_kernel_map_.count(key) != 0)
      throw std::runtime_error("Kernel already registered: " + key.second + " on device " +
                               std::to_string(static_cast<int>(key.first)));
    key_to_kernel_map_.emplace(key, KernelFunction(std::forward<FuncT>(kernel)));
  }

 private:
  std::map<KeyT, KernelFunction> key_to_kernel_map_;
};

namespace detail {
struct KernelRegistrar {
  template <typename FuncT>
  KernelRegistrar(DeviceType device, const char* name, FuncT&& fn) {
    Dispatcher::Instance().Register({device, name}, std::forward<FuncT>(fn));
  }
};
}  // namespace detail

}  // namespace infini_train

#define TITB_CONCAT_IMPL(a, b) a##b
#define TITB_CONCAT(a, b) TITB_CONCAT_IMPL(a, b)
// Registers `kernel_func` under #kernel_name for `device` when the enclosing scope is initialised:
// at namespace scope that is static initialisation, inside a function the first time control
// passes over the statement.
#define REGISTER_KERNEL(device, kernel_name, kernel_func)                                            \
  static ::infini_train::detail::KernelRegistrar TITB_CONCAT(_titb_kernel_registrar_, __COUNTER__)( \
      device, #kernel_name, kernel_func)

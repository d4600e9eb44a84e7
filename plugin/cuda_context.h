// SPDX-License-Identifier: Apache-2.0
/**
 * @file  cuda_context.h
 * @brief nntrainer::Context for the CUDA backend, loadable at run time the way the reference loads any external
 *        context: Engine::registerContext(library, base) (nntrainer/engine.cpp:138-171) dlopens the library, looks up
 *        `ml_train_context_pluggable` (nntrainer/context.h:225-240), calls its createfunc and registers the result
 *        under getName().
 *
 * The context answers to the name "gpu": per-layer routing goes through parseComputeEngine, which knows only
 * cpu / gpu / qnn (nntrainer/engine.cpp:64-84), so with OpenCL disabled a layer opts in with `engine=gpu` and no line
 * of the reference changes. It keeps its own factory map like ClContext does (nntrainer/cl_context.h:96-205) and
 * overrides BOTH createLayerObject overloads (nntrainer/context.h:116-140; the base versions return nullptr). The
 * layers it hands out are the stock ones: a fully connected layer created here forwards through
 * Tensor::dot -> FloatTensor::dotQnK, where the ENABLE_CUDA branch calls cuda_backend.
 * Engine::registerContext dereferences getMemAllocator() (nntrainer/engine.h:82-84) and keeps it under the context's
 * name, so the constructor installs one: CudaHostAllocator, whose memory is page-locked and device-mapped, so that a
 * decode call on tensors planned into it needs no copy-engine transfer and no stream synchronisation.
 */
#ifndef NNTR_CUDA_CONTEXT_H_
#define NNTR_CUDA_CONTEXT_H_

#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include <context.h>
#include <layer_devel.h>
#include <mem_allocator.h>

namespace nntrainer {

/** MemAllocator (nntrainer/mem_allocator.h:25-32) over nntr_cuda_host_alloc / nntr_cuda_host_free */
class CudaHostAllocator : public MemAllocator {
public:
  /** @throws std::bad_alloc when the driver refuses (no device bound yet, or out of page-locked memory) */
  void alloc(void **ptr, size_t size, size_t alignment) override;
  void free(void *ptr) override;
  std::string getName() override { return "gpu"; }
};

class CudaContext : public Context {
public:
  CudaContext();
  ~CudaContext() override = default;

  /** binds the CUDA device and registers the default layer factories; ML_ERROR_NONE (0) or a negative ML_ERROR_* */
  int init() override;

  std::string getName() override { return "gpu"; }

  PtrType<nntrainer::Layer> createLayerObject(const std::string &type,
                                              const std::vector<std::string> &props = {}) override;
  PtrType<nntrainer::Layer> createLayerObject(const int int_key, const std::vector<std::string> &props = {}) override;

  /** registers a layer factory under a string key and an integer key (-1: none); returns the integer key.
   *  Throws std::invalid_argument when either key is taken (as ClContext::registerFactory does). */
  int registerFactory(const FactoryType<nntrainer::Layer> factory, const std::string &key, const int int_key = -1);

  /** true once init() has bound a device */
  bool ready() const { return ready_; }

private:
  std::mutex mutex_;
  std::unordered_map<std::string, FactoryType<nntrainer::Layer>> by_name_;
  std::unordered_map<int, std::string> by_int_;
  bool ready_ = false;
};

} // namespace nntrainer

#endif /* NNTR_CUDA_CONTEXT_H_ */

// SPDX-License-Identifier: Apache-2.0
/**
 * @file  cuda_context.cpp
 * @brief The run-time plug-in: CudaContext and the `ml_train_context_pluggable` symbol the Engine looks up
 *        (nntrainer/context.h:225-240, nntrainer/engine.cpp:138-171).
 */
#include "cuda_context.h"

#include <algorithm>
#include <new>
#include <stdexcept>

#include <fc_layer.h>
#include <nntrainer_error.h>
#include <nntrainer_log.h>

#include "../include/nntr_cuda.h"
#include "cuda_backend.h"

namespace nntrainer {

void CudaHostAllocator::alloc(void **ptr, size_t size, size_t alignment) {
  // page-locked memory starts on a page boundary, which satisfies every alignment the framework asks for
  if (!ptr || (alignment & (alignment - 1)) || alignment > 4096)
    throw std::invalid_argument("cuda_context: unsupported allocation request");
  if (nntr_cuda_host_alloc(ptr, size ? size : 1) != NNTR_CUDA_OK) {
    ml_loge("cuda_context: %s", nntr_cuda_last_error());
    throw std::bad_alloc();
  }
}

void CudaHostAllocator::free(void *ptr) {
  if (nntr_cuda_host_free(ptr) != NNTR_CUDA_OK)
    ml_loge("cuda_context: %s", nntr_cuda_last_error());
}

CudaContext::CudaContext() : Context(std::make_shared<ContextData>()) {
  // host-side allocator for whatever the framework plans on this context's behalf; device memory is managed inside
  // libnntr_cuda.so (weights are mirrored into HBM when they are registered)
  getContextData()->setMemAllocator(std::make_shared<CudaHostAllocator>());
}

int CudaContext::init() {
  const int rc = nntr_cuda_init(0);
  if (rc != NNTR_CUDA_OK) {
    ml_loge("cuda_context: %s", nntr_cuda_last_error());
    return rc == NNTR_CUDA_ERR_UNSUPPORTED ? ML_ERROR_NOT_SUPPORTED : ML_ERROR_INVALID_PARAMETER;
  }
  try {
    // the same registration call ClContext::add_default_object makes (nntrainer/cl_context.cpp:92-96), with the stock
    // layer class: its forwarding reaches the GPU through Tensor::dot
    registerFactory(nntrainer::createLayer<FullyConnectedLayer>, FullyConnectedLayer::type,
                    ml::train::LayerType::LAYER_FC);
  } catch (std::exception &e) {
    ml_loge("cuda_context: registering layers failed, reason: %s", e.what());
    return ML_ERROR_INVALID_PARAMETER;
  }
  ready_ = true;
  return ML_ERROR_NONE;
}

int CudaContext::registerFactory(const FactoryType<nntrainer::Layer> factory, const std::string &key, const int int_key) {
  std::string lower = key;
  std::transform(lower.begin(), lower.end(), lower.begin(), [](unsigned char c) { return std::tolower(c); });
  std::lock_guard<std::mutex> lk(mutex_);
  if (by_name_.count(lower))
    throw std::invalid_argument("cuda_context: layer key is already registered: " + key);
  int assigned = int_key;
  if (assigned == -1) {
    assigned = 0x10000; // keys handed out here start above the predefined layer types
    while (by_int_.count(assigned))
      ++assigned;
  } else if (by_int_.count(assigned)) {
    throw std::invalid_argument("cuda_context: integer key is already registered: " + std::to_string(int_key));
  }
  by_name_[lower] = factory;
  by_int_[assigned] = lower;
  return assigned;
}

Context::PtrType<nntrainer::Layer> CudaContext::createLayerObject(const std::string &type,
                                                                  const std::vector<std::string> &props) {
  std::string lower = type;
  std::transform(lower.begin(), lower.end(), lower.begin(), [](unsigned char c) { return std::tolower(c); });
  FactoryType<nntrainer::Layer> f;
  {
    std::lock_guard<std::mutex> lk(mutex_);
    auto it = by_name_.find(lower);
    if (it == by_name_.end())
      throw exception::not_supported("cuda_context: unknown layer type " + type);
    f = it->second;
  }
  return f(props);
}

Context::PtrType<nntrainer::Layer> CudaContext::createLayerObject(const int int_key,
                                                                  const std::vector<std::string> &props) {
  std::string name;
  {
    std::lock_guard<std::mutex> lk(mutex_);
    auto it = by_int_.find(int_key);
    if (it == by_int_.end())
      throw exception::not_supported("cuda_context: unknown layer key " + std::to_string(int_key));
    name = it->second;
  }
  return createLayerObject(name, props);
}

} // namespace nntrainer

static nntrainer::Context *create_cuda_context() {
  auto *c = new nntrainer::CudaContext();
  c->init(); // a failed init is logged; the Engine still gets a named context whose layers cannot be created
  return c;
}
static void destroy_cuda_context(nntrainer::Context *c) { delete c; }

extern "C" {
nntrainer::ContextPluggable ml_train_context_pluggable{create_cuda_context, destroy_cuda_context};
}

// SPDX-License-Identifier: Apache-2.0
/**
 * @file  context_probe.cpp
 * @brief Test harness: loads libcuda_context.so the way Engine::registerContext does (nntrainer/engine.cpp:138-171:
 *        dlopen with RTLD_LAZY | RTLD_LOCAL, dlsym "ml_train_context_pluggable", createfunc()), and prints what the
 *        Engine would see. It is built together with the reference's own mem_allocator.cpp, so the one data symbol the
 *        plug-in needs from the framework at load time (the MemAllocator vtable) resolves; the framework's logger is a
 *        stub. Used by tests/test_plugin.py; not part of the library.
 */
#include <cstdarg>
#include <cstdio>
#include <dlfcn.h>
#include <stdexcept>
#include <string>

#include <context.h>
#include <nntrainer_error.h>
#include <nntrainer_logger.h>

/* the framework's logger (nntrainer/nntrainer_logger.h:152): swallowed here */
void __nntrainer_log_print(nntrainer_loglevel, const std::string, ...) {}

int main(int argc, char **argv) {
  if (argc != 2) {
    fprintf(stderr, "usage: %s <libcuda_context.so>\n", argv[0]);
    return 2;
  }
  void *handle = dlopen(argv[1], RTLD_LAZY | RTLD_LOCAL);
  if (!handle) {
    fprintf(stderr, "dlopen: %s\n", dlerror());
    return 3;
  }
  auto *pluggable = reinterpret_cast<nntrainer::ContextPluggable *>(dlsym(handle, "ml_train_context_pluggable"));
  if (!pluggable) {
    fprintf(stderr, "dlsym: %s\n", dlerror());
    return 4;
  }
  nntrainer::Context *ctx = pluggable->createfunc();
  if (!ctx)
    return 5;
  printf("name=%s\n", ctx->getName().c_str());
  printf("mem_allocator=%s\n", ctx->getMemAllocator() ? ctx->getMemAllocator()->getName().c_str() : "null");
  bool unknown_rejected = false;
  try {
    auto l = ctx->createLayerObject("no_such_layer", {});
  } catch (const nntrainer::exception::not_supported &) {
    unknown_rejected = true;
  }
  printf("unknown_layer_rejected=%d\n", unknown_rejected ? 1 : 0);
  bool unknown_key_rejected = false;
  try {
    auto l = ctx->createLayerObject(987654, {});
  } catch (const std::invalid_argument &) {
    unknown_key_rejected = true;
  }
  printf("unknown_key_rejected=%d\n", unknown_key_rejected ? 1 : 0);
  pluggable->destroyfunc(ctx);
  return 0;
}

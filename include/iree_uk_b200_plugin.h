/*
 * iree_uk_b200_plugin.h - what libiree_uk_b200_plugin.so exports beside the reference's
 * iree_hal_executable_plugin_query (runtime/src/iree/hal/local/executable_plugin.h:186-198).
 * The plugin resolves the imports iree_uk_mmt4d, iree_uk_pack and iree_uk_unpack of compiled
 * IREE code to libiree_uk_b200.so. The two calls below let the runtime that loaded it - which
 * owns the CUDA stream - tell it where to enqueue. No counterpart in the reference.
 */
#ifndef IREE_UK_B200_PLUGIN_H_
#define IREE_UK_B200_PLUGIN_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Sets the CUDA stream the resolved imports enqueue on and, optionally, device scratch for
 * mmt4d (256-byte aligned; NULL / 0 for none: mmt4d then uses the library's static scratch or
 * its scratch-free kernels). `self` is the value the plugin's load() returned. Not thread-safe
 * against import calls in flight on other host threads. Returns an iree_uk_b200_status_t. */
int iree_uk_b200_plugin_configure(void* self, void* cu_stream, void* workspace,
                                  size_t workspace_bytes);

/* The library status of the last import call that failed since the previous query (0: none),
 * cleared by the call: an import thunk can only return "non-zero", this says why. */
int iree_uk_b200_plugin_last_status(void* self);

#ifdef __cplusplus
} /* extern "C" */
#endif

#endif /* IREE_UK_B200_PLUGIN_H_ */

/*
 * iree_uk_b200_plugin.c - an IREE executable plugin that resolves the three ukernel imports
 * iree_uk_mmt4d, iree_uk_pack and iree_uk_unpack to libiree_uk_b200.so.
 *
 * The plugin interface is the reference's own: this file includes its standalone header
 * (runtime/src/iree/hal/local/executable_plugin.h:386-461, v0 interface) from a reference
 * checkout at build time and copies nothing from it. The pattern follows
 * samples/custom_dispatch/cpu/plugin/system_plugin.c:62-97 (import thunk) and :147-209
 * (load / unload / resolve / query).
 *
 * What an import call looks like: compiled code calls every import as
 *     int fn(void* params_ptr, void* context, void* reserved)
 * where params_ptr points at the packed operands of the iree_codegen.ukernel.generic op in
 * native alignment (compiler/src/iree/compiler/Codegen/Dialect/Codegen/IR/UKernelOps.cpp:113-145:
 * each memref as base pointer, offset and its strided outer strides, then the scalars) followed
 * by the processor_data pointer that "hal.import.fields" asks for
 * (Codegen/Common/CPU/CPULowerToUKernels.cpp:104-111). For mmt4d that is lhs, rhs, out with one
 * stride each, then M, N, K, M0, N0, K0, flags (CPULowerToUKernels.cpp:256-260); for pack and
 * unpack two strides per memref and the sizes, padding value and flags (:378-383, :466-471).
 * Field for field these are iree_uk_mmt4d_params_t, iree_uk_pack_params_t and
 * iree_uk_unpack_params_t, so a thunk hands params_ptr to the library as it is; the layouts
 * are asserted below.
 *
 * What differs from a CPU plugin: the buffers the thunks receive must be device pointers and
 * the work is enqueued on a CUDA stream, so the runtime that loads this plugin has to tell it
 * which stream, and may give it scratch memory. Both arrive as plugin parameters at load
 * ("stream", "workspace", "workspace_bytes": decimal or 0x-prefixed integers) or later through
 * iree_uk_b200_plugin_configure. Without a workspace the mmt4d thunk uses the library's
 * static-scratch entry point; when a problem does not fit that array it falls back to the
 * scratch-free kernels (an import call has no allocator to turn to) unless the runtime that
 * loaded the plugin allowed stream-ordered allocation with the parameter "scratch_pool" = 1,
 * in which case the scratch comes from the library's own memory pool on the call's stream.
 *
 * A thunk returns 0 on success and the library's status code otherwise.
 */
#include <stddef.h>
#include <stdint.h>

#include "iree/hal/local/executable_plugin.h"
#include "iree_uk_b200.h"
#include "iree_uk_b200_plugin.h"

_Static_assert(sizeof(iree_uk_mmt4d_params_t) == 9 * 8 + 3 * 8 + 4 * 4 + 8, "mmt4d operand packing");
_Static_assert(offsetof(iree_uk_mmt4d_params_t, M) == 72, "mmt4d operand packing");
_Static_assert(offsetof(iree_uk_mmt4d_params_t, cpu_data) == 112, "mmt4d operand packing");
_Static_assert(sizeof(iree_uk_pack_params_t) == 8 * 8 + 6 * 8 + 8 + 8 + 8, "pack operand packing");
_Static_assert(offsetof(iree_uk_pack_params_t, in_size0) == 64, "pack operand packing");
_Static_assert(offsetof(iree_uk_pack_params_t, cpu_data) == 128, "pack operand packing");
_Static_assert(sizeof(iree_uk_unpack_params_t) == 8 * 8 + 6 * 8 + 8 + 8, "unpack operand packing");
_Static_assert(offsetof(iree_uk_unpack_params_t, in_size0) == 64, "unpack operand packing");
_Static_assert(offsetof(iree_uk_unpack_params_t, cpu_data) == 120, "unpack operand packing");

typedef struct plugin_state_t {
  iree_hal_executable_plugin_allocator_t host_allocator;
  void* stream;            /* CUstream every call is enqueued on */
  void* workspace;         /* device scratch for mmt4d, or NULL */
  size_t workspace_bytes;
  int scratch_pool;        /* nonzero: problems beyond the static scratch may use the library's pool */
  int last_status;         /* library status of the last failing call, 0 when none failed */
} plugin_state_t;

/* ---- import thunks ---- */

static int mmt4d_thunk(void* params_ptr, void* context, void* reserved) {
  (void)reserved;
  plugin_state_t* st = (plugin_state_t*)context;
  const iree_uk_mmt4d_params_t* p = (const iree_uk_mmt4d_params_t*)params_ptr;
  int rc;
  if (st->workspace && st->workspace_bytes >= iree_uk_b200_mmt4d_workspace_size(p)) {
    rc = iree_uk_b200_mmt4d_ws(p, st->workspace, st->workspace_bytes, st->stream);
  } else {
    rc = iree_uk_b200_mmt4d_static_scratch(p, st->stream);
    if (rc == IREE_UK_B200_WORKSPACE_TOO_SMALL)
      rc = st->scratch_pool ? iree_uk_b200_mmt4d_pooled(p, st->stream) : iree_uk_b200_mmt4d(p, st->stream);
  }
  if (rc) st->last_status = rc;
  return rc;
}

static int pack_thunk(void* params_ptr, void* context, void* reserved) {
  (void)reserved;
  plugin_state_t* st = (plugin_state_t*)context;
  const int rc = iree_uk_b200_pack((const iree_uk_pack_params_t*)params_ptr, st->stream);
  if (rc) st->last_status = rc;
  return rc;
}

static int unpack_thunk(void* params_ptr, void* context, void* reserved) {
  (void)reserved;
  plugin_state_t* st = (plugin_state_t*)context;
  const int rc = iree_uk_b200_unpack((const iree_uk_unpack_params_t*)params_ptr, st->stream);
  if (rc) st->last_status = rc;
  return rc;
}

/* ---- parameters ---- */

static int view_equals(iree_hal_executable_plugin_string_view_t v, const char* s) {
  size_t i = 0;
  for (; i < v.size; ++i)
    if (s[i] == '\0' || s[i] != v.data[i]) return 0;
  return s[i] == '\0';
}

/* Decimal or 0x-prefixed hexadecimal; returns 0 on a malformed or empty value. */
static int parse_u64(iree_hal_executable_plugin_string_view_t v, uint64_t* out) {
  uint64_t x = 0;
  size_t i = 0;
  if (v.size == 0) return 0;
  if (v.size > 2 && v.data[0] == '0' && (v.data[1] == 'x' || v.data[1] == 'X')) {
    for (i = 2; i < v.size; ++i) {
      const char c = v.data[i];
      uint64_t d;
      if (c >= '0' && c <= '9') d = (uint64_t)(c - '0');
      else if (c >= 'a' && c <= 'f') d = (uint64_t)(c - 'a' + 10);
      else if (c >= 'A' && c <= 'F') d = (uint64_t)(c - 'A' + 10);
      else return 0;
      x = (x << 4) | d;
    }
  } else {
    for (i = 0; i < v.size; ++i) {
      if (v.data[i] < '0' || v.data[i] > '9') return 0;
      x = x * 10 + (uint64_t)(v.data[i] - '0');
    }
  }
  *out = x;
  return 1;
}

/* ---- plugin interface ---- */

static iree_hal_executable_plugin_status_t plugin_load(
    const iree_hal_executable_plugin_environment_v0_t* environment, size_t param_count,
    const iree_hal_executable_plugin_string_pair_t* params, void** out_self) {
  plugin_state_t* st = NULL;
  iree_hal_executable_plugin_status_t status = iree_hal_executable_plugin_allocator_malloc(
      environment->host_allocator, sizeof(*st), (void**)&st);
  if (status) return status;
  st->host_allocator = environment->host_allocator;
  st->stream = NULL;
  st->workspace = NULL;
  st->workspace_bytes = 0;
  st->scratch_pool = 0;
  st->last_status = 0;
  for (size_t i = 0; i < param_count; ++i) {
    uint64_t v = 0;
    const int known = view_equals(params[i].key, "stream") ? 1
                      : view_equals(params[i].key, "workspace") ? 2
                      : view_equals(params[i].key, "workspace_bytes") ? 3
                      : view_equals(params[i].key, "scratch_pool") ? 4 : 0;
    if (!known) continue; /* parameters meant for other plugins */
    if (!parse_u64(params[i].value, &v)) {
      iree_hal_executable_plugin_allocator_free(environment->host_allocator, st);
      return iree_hal_executable_plugin_status_from_code(
          IREE_HAL_EXECUTABLE_PLUGIN_STATUS_INVALID_ARGUMENT);
    }
    if (known == 1) st->stream = (void*)(uintptr_t)v;
    if (known == 2) st->workspace = (void*)(uintptr_t)v;
    if (known == 3) st->workspace_bytes = (size_t)v;
    if (known == 4) st->scratch_pool = v != 0;
  }
  *out_self = st;
  return iree_hal_executable_plugin_ok_status();
}

static void plugin_unload(void* self) {
  plugin_state_t* st = (plugin_state_t*)self;
  iree_hal_executable_plugin_allocator_free(st->host_allocator, st);
}

static iree_hal_executable_plugin_status_t plugin_resolve(
    void* self, const iree_hal_executable_plugin_resolve_params_v0_t* params,
    iree_hal_executable_plugin_resolution_t* out_resolution) {
  static const struct {
    const char* name;
    int (*fn)(void*, void*, void*);
  } table[] = {
      {"iree_uk_mmt4d", mmt4d_thunk},
      {"iree_uk_pack", pack_thunk},
      {"iree_uk_unpack", unpack_thunk},
  };
  *out_resolution = 0;
  int required_missing = 0;
  for (size_t i = 0; i < params->count; ++i) {
    if (params->out_fn_ptrs[i]) continue; /* resolved by an earlier provider */
    const char* name = params->symbol_names[i];
    const int optional = iree_hal_executable_plugin_import_is_optional(name);
    if (optional) ++name;
    int found = 0;
    for (size_t j = 0; j < sizeof(table) / sizeof(table[0]); ++j) {
      if (iree_hal_executable_plugin_strcmp(name, table[j].name) == 0) {
        params->out_fn_ptrs[i] = (void*)table[j].fn;
        params->out_fn_contexts[i] = self;
        found = 1;
        break;
      }
    }
    if (found) continue;
    if (optional) *out_resolution |= IREE_HAL_EXECUTABLE_PLUGIN_RESOLUTION_MISSING_OPTIONAL;
    else required_missing = 1;
  }
  return required_missing ? iree_hal_executable_plugin_status_from_code(
                                IREE_HAL_EXECUTABLE_PLUGIN_STATUS_NOT_FOUND)
                          : iree_hal_executable_plugin_ok_status();
}

IREE_HAL_EXECUTABLE_PLUGIN_EXPORT const iree_hal_executable_plugin_header_t**
iree_hal_executable_plugin_query(iree_hal_executable_plugin_version_t max_version, void* reserved) {
  (void)reserved;
  static const iree_hal_executable_plugin_header_t header = {
      .version = IREE_HAL_EXECUTABLE_PLUGIN_VERSION_LATEST,
      .name = "iree_uk_b200",
      .description = "mmt4d / pack / unpack ukernels on B200 (sm_100a) through libiree_uk_b200.so",
      /* not STANDALONE: the thunks call into the CUDA runtime */
      .features = IREE_HAL_EXECUTABLE_PLUGIN_FEATURE_NONE,
      .sanitizer = IREE_HAL_EXECUTABLE_PLUGIN_SANITIZER_KIND,
  };
  static const iree_hal_executable_plugin_v0_t plugin = {
      .header = &header,
      .load = plugin_load,
      .unload = plugin_unload,
      .resolve = plugin_resolve,
  };
  return max_version >= IREE_HAL_EXECUTABLE_PLUGIN_VERSION_0_1
             ? (const iree_hal_executable_plugin_header_t**)&plugin
             : NULL;
}

/* ---- configuration after load ---- */

IREE_HAL_EXECUTABLE_PLUGIN_EXPORT int iree_uk_b200_plugin_configure(void* self, void* cu_stream,
                                                                    void* workspace,
                                                                    size_t workspace_bytes) {
  plugin_state_t* st = (plugin_state_t*)self;
  if (!st || (workspace_bytes && !workspace)) return IREE_UK_B200_INVALID_ARGUMENT;
  st->stream = cu_stream;
  st->workspace = workspace;
  st->workspace_bytes = workspace_bytes;
  return IREE_UK_B200_OK;
}

IREE_HAL_EXECUTABLE_PLUGIN_EXPORT int iree_uk_b200_plugin_last_status(void* self) {
  plugin_state_t* st = (plugin_state_t*)self;
  if (!st) return IREE_UK_B200_INVALID_ARGUMENT;
  const int rc = st->last_status;
  st->last_status = 0;
  return rc;
}

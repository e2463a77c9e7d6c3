/*
 * iree_uk_b200_testing.h - hooks of libiree_uk_b200.so that exist for its own tests. They are
 * exported so that the tests can reach them through the C ABI like everything else; a caller
 * of the library has no use for them. No counterpart in the reference.
 */
#ifndef IREE_UK_B200_TESTING_H_
#define IREE_UK_B200_TESTING_H_

#include "iree_uk_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Failure detection without a GPU fault. While enabled (process-wide), the producers of the
 * tensor-core mmt4d kernels (the TMA warp, the re-tiling warps) issue nothing, so the waits of
 * the other roles run out; the limit of every device-side wait drops from about a second to a
 * few tens of milliseconds for such launches. The kernels must then record the timeout
 * (iree_uk_b200_device_status returns IREE_UK_B200_DEVICE_TIMEOUT), return, and leave the
 * context usable. Returns the previous setting. */
IREE_UK_B200_EXPORT int iree_uk_b200_testing_starve_producers(int enable);

/* Runs a tensor-core mmt4d (arguments as iree_uk_b200_mmt4d_ws) on one given kernel form
 * instead of the form the library would choose by problem size, so that every form can be
 * checked on small problems. IREE_UK_B200_UNSUPPORTED when the problem is not a tensor-core
 * problem or the form cannot run it. */
#define IREE_UK_B200_TESTING_FORM_TWO_CTA 5          /* CTA pairs, whole re-tile in the pre-pass */
#define IREE_UK_B200_TESTING_FORM_ONE_CTA 6          /* one CTA per tile */
#define IREE_UK_B200_TESTING_FORM_TWO_CTA_STREAMED 7 /* CTA pairs, re-tile finished by the kernel */
IREE_UK_B200_EXPORT int iree_uk_b200_testing_mmt4d_form(const iree_uk_mmt4d_params_t* params,
                                                        void* workspace, size_t workspace_bytes,
                                                        int form, void* cu_stream);

#ifdef __cplusplus
} /* extern "C" */
#endif

#endif /* IREE_UK_B200_TESTING_H_ */

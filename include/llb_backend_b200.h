/* llb_backend_b200.h -- the reference's backend surface (host/llb_backend.h:7-34) on libllb_b200.so.
 *
 * host/llb_backend.h asks that "a backend header comes first and defines, macro- or static-inline-thin" the names
 * below; the reference's own is host/llb_backend_cuda.h.  This header takes that header's place in a build against
 * libllb_b200.so: include it INSTEAD of llb_backend_cuda.h, then host/llb_backend.h.  Same names, same argument
 * meaning, and the reference's truth sense: bool results, true = queued / done, llb_alloc_zero returns 0 on failure.
 *
 *   llb_dptr                                   host/llb_backend_cuda.h:5 (an unsigned 64-bit device address; offsets add)
 *   LLB_LAUNCH, LLB_LAUNCH_SM                  host/llb_backend_cuda.h:7-11
 *   llb_graph_begin / _end / _bail             host/llb_backend_cuda.h:125-184
 *   llb_alloc_zero llb_zero llb_read llb_copy llb_write llb_sync llb_dev    host/llb_backend_cuda.h:186-221
 *
 * Kernel handles: the reference fetches CUfunction handles by name from its NVRTC module
 * (tools/payload-spec.patch:9-23).  Here a handle is `llb_kernel` = llb_b200_kernel_by_name(name); a name the library
 * does not export gives NULL, and LLB_LAUNCH on a NULL handle returns false without queueing anything, which the
 * reference's chains turn into err_fail("device launch failed").
 */
#ifndef LLB_BACKEND_B200_H
#define LLB_BACKEND_B200_H
#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#include "llb_b200.h"

typedef llb_b200_dptr llb_dptr;
typedef const llb_b200_kernel *llb_kernel;

#define LLB_LAUNCH(k, gx, gy, bx, ...) LLB_LAUNCH_SM(k, gx, gy, bx, 0, __VA_ARGS__)
#define LLB_LAUNCH_SM(k, gx, gy, bx, sm, ...) ({ \
  void *a_[] = { __VA_ARGS__ }; \
  llb_b200_launch((k), (unsigned)(gx), (unsigned)(gy), (unsigned)(bx), (unsigned)(sm), a_, (unsigned)(sizeof a_ / sizeof *a_)) == 0; })

static inline llb_kernel llb_kernel_by_name(const char *name) { return llb_b200_kernel_by_name(name); }
static inline void llb_graph_begin(void) { llb_b200_graph_begin(); }
static inline void llb_graph_end(void) { llb_b200_graph_end(); }
static inline void llb_graph_bail(void) { llb_b200_graph_bail(); }

static inline llb_dptr llb_alloc_zero(size_t bytes) { return llb_b200_alloc_zero(bytes); }
static inline bool llb_zero(llb_dptr p, size_t bytes) { return llb_b200_zero(p, bytes) == 0; }
static inline bool llb_read(void *h, llb_dptr p, size_t bytes) { return llb_b200_read(h, p, bytes) == 0; }
static inline bool llb_copy(llb_dptr d, llb_dptr s, size_t bytes) { return llb_b200_copy(d, s, bytes) == 0; }
static inline bool llb_write(llb_dptr d, const void *h, size_t bytes) { return llb_b200_write(d, h, bytes) == 0; }
static inline bool llb_sync(void) { return llb_b200_sync() == 0; }
/* the reference's corpus lives in unified memory, so a host pointer's bits are its device address
 * (host/llb_backend_cuda.h:221); the same holds here for memory the caller registered or allocated as managed */
#define llb_dev(p) ((llb_dptr)(uintptr_t)(p))
#endif

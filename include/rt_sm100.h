/* rt_sm100.h -- the B200 runtime as a run-side descriptor for Booth's src/exec.
 *
 * The reference defines one descriptor per run target (rt_desc_t,
 * src/exec/exec.h:69-93) and a registration list that is still empty
 * (src/exec/execs.c:7-11); porting a launcher to that contract is its stated next
 * step (docs/roadmap.md:15-18). libbooth_sm100 exports such a descriptor:
 *
 *     extern const rt_desc_t rt_sm100;          name "sm100", artefact "cubin"
 *
 * so registering the B200 is one line in src/exec/execs.c:
 *
 *     const rt_desc_t * const rt_list[] = { &rt_sm100, NULL };
 *
 * When the reference's exec.h has been included first its types are used as they
 * are. Otherwise this header declares the same interface (same field order and
 * types, hence the same layout), so the descriptor can be used on its own. */
#ifndef RT_SM100_H
#define RT_SM100_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef BOOTH_EXEC_H

/* Status codes of the contract (src/exec/exec.h:12-20). */
#define RT_OK        0
#define RT_ENODRV   -1
#define RT_ESYM     -2
#define RT_EDRV     -3
#define RT_ENODEV   -4
#define RT_EIO      -5
#define RT_EKERN    -6
#define RT_EUNSUP   -7
#define RT_EINPUT   -8

typedef uint64_t rt_ptr;                              /* device address, 0 = null */

typedef struct { const void *p; uint32_t size; } rt_arg_t;     /* one kernel argument */

#define RT_DEV_MAX   1024                             /* caller-held handle bytes */
#define RT_KERN_MAX   192

typedef struct { uint32_t grid[3]; uint32_t block[3]; uint32_t shmem; } rt_dim_t;

typedef struct rt_desc {
    const char *name;
    const char *artefact;
    uint32_t    dev_size;
    uint32_t    kern_size;
    int    (*open)  (void *dev);
    void   (*shut)  (void *dev);
    int    (*load)  (void *dev, const char *path, const char *kern, void *out);
    void   (*unload)(void *dev, void *kern);
    rt_ptr (*alloc) (void *dev, size_t n);
    void   (*dfre)  (void *dev, rt_ptr p);
    int    (*h2d)   (void *dev, rt_ptr dst, const void *src, size_t n);
    int    (*d2h)   (void *dev, void *dst, rt_ptr src, size_t n);
    int    (*run)   (void *dev, const void *kern, const rt_dim_t *dim,
                     const rt_arg_t *args, uint32_t nargs);
    int    (*sync)  (void *dev);
    int    (*hmap)  (void *dev, void **hp, rt_ptr *dp, size_t n);
    void   (*hfre)  (void *dev, void *hp);
    void   (*trak)  (void *dev, rt_ptr p, size_t n, const char *lbl, int fl);
    const char *(*errs)(int rc);
} rt_desc_t;

#endif /* BOOTH_EXEC_H */

/* All ten required operations and the four optional ones. run only enqueues,
 * sync waits (src/exec/exec.h:105-106). dev_size and kern_size fit the
 * caller-held handles (16 and 176 bytes). */
extern const rt_desc_t rt_sm100;

#ifdef __cplusplus
}
#endif
#endif /* RT_SM100_H */

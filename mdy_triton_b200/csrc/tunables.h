/* Ids of the integer knobs behind mdy_set_tunable / mdy_get_tunable.  Internal to the library and its
 * tests and tuning scripts (mirrored in mdy_triton_b200/_C/__init__.py); a value of 0 means "built-in
 * default" for every knob. */
#pragma once

#define MDY_TUNE_CE_THREADS 0           /* threads per CTA of the row-per-CTA cross-entropy kernels (default: by row length) */
#define MDY_TUNE_CE_FUSED_CTAS_PER_SM 1 /* resident CTAs per SM the row-per-CTA one-pass kernel is limited to */
#define MDY_TUNE_NORM_CTAS_PER_SM 2     /* persistent-grid width of the norm kernels, in CTAs per SM */
#define MDY_TUNE_SWIGLU_UNROLL 3        /* 16-byte vectors per thread in SwiGLU (1, 2 or 4) */
#define MDY_TUNE_CE_FUSED_IMPL 4        /* 0 auto (cluster kernel; row-per-CTA kernel for shapes it rejects), 1 row-per-CTA always */
#define MDY_TUNE_ROPE_THREADS 5         /* threads per CTA of the RoPE kernel */
#define MDY_TUNE_CE_CLUSTER_SLICE_KB 6  /* largest slice of a row one CTA of the cluster kernel stages (KiB) */
#define MDY_TUNE_CE_CLUSTER_THREADS 7   /* threads per CTA of the cluster kernel; with ids 8 and 15 selects a compiled shape:
                                           (threads, vectors, CTAs/SM) = (256,4,3) (256,8,2) (512,2,2) (512,4,1) (1024,2,1) */
#define MDY_TUNE_CE_CLUSTER_VPC 8       /* 16-byte vectors per thread per chunk there */
#define MDY_TUNE_CE_WAIT_TEST 9         /* test hook of the cluster kernel's bounded waits: k > 0 makes a wait give up after
                                           2^10 tries (about a millisecond) and leaves the first chunk of the first row of
                                           the first k clusters unrequested, so that wait runs out */
#define MDY_TUNE_ROPE_HEADS_PER_THREAD 10 /* heads a RoPE thread rotates per work item: 1, 2 or 4 */
#define MDY_TUNE_ROPE_GRID_PER_SM 11    /* cap of the RoPE grid, in CTAs per SM (grid-stride loop) */
#define MDY_TUNE_NORM_BWD_THREADS 12    /* CTA size the norm backward aims for: 128, 256 or 512 */
#define MDY_TUNE_NORM_FWD_VPT 13        /* 16-byte vectors per thread the norm forward plans for: 1, 2, 4 */
#define MDY_TUNE_NORM_BWD_VPT 14        /* the same for the norm backward */
#define MDY_TUNE_CE_CLUSTER_MINB 15     /* CTAs per SM that shape is compiled for (register cap) */
#define MDY_TUNE_NORM_POW2_GROUPS 16    /* 1: threads per row rounded up to a power of two instead of a warp multiple */
#define MDY_TUNE_NORM_FWD_GROUP 17      /* threads per row of the norm forward (rounded up to a warp multiple) */
#define MDY_TUNE_NORM_BWD_GROUP 18      /* the same for the norm backward */
#define MDY_TUNE_NORM_FWD_THREADS 19    /* CTA size the norm forward aims for: 128, 256 or 512 */
#define MDY_TUNE_NORM_IMPL 20           /* 0 choose, 1 register-resident norm kernels always, 2 shared-memory-staged wherever possible */
#define MDY_TUNE_CE_VP_CTAS_PER_SM 21   /* CTAs per SM of the one-kernel vocab-parallel cross-entropy */
#define MDY_TUNE_CE_VP_SLOTS 22         /* its shared-memory slots per CTA (3 or 4) */
#define MDY_TUNE_CE_VP_SLICE_KB 23       /* largest column slice of the one-kernel vocab-parallel cross-entropy (KiB, default 32) */
#define MDY_TUNE_NORM_TEAM 24           /* staged norm kernels: warps per row (1, 2 or 4; 0 = choose) */
#define MDY_TUNE_COUNT 25

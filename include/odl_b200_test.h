/*
 * odl_b200_test -- kernel-selection overrides of libodl_b200.so, for test programs only.
 *
 * The launchers of the library choose tile widths, split-K forms, CTA pairing and the conv algorithm from the problem
 * size.  Parity tests need every one of those code paths on small shapes the automatic choice would never send there,
 * so the library exports these setters.  They write PROCESS-GLOBAL ints that the launchers read without locking: call
 * them from the one thread that also issues the library calls, and reset each to 0 (automatic) afterwards.  A product
 * host has no reason to call them; none has a counterpart in the reference (its one run-time kernel switch is the
 * ORIGIN_KERNEL_ALGO environment variable, src/utils/env_config.cpp:14-36).  All return ODL_OK.
 */
#ifndef ODL_B200_TEST_H_
#define ODL_B200_TEST_H_

#ifdef __cplusplus
extern "C" {
#endif

/* GEMM column-tile width: 64, 128 or 256; 0 = automatic. */
int odl_debug_set_tile_n(int bn);
/* K-blocks of 32 accumulated in TMEM between two drains into registers; 0 = automatic (2 in 3xTF32). */
int odl_debug_set_chunk(int chunk_kb);
/* Split-K: 1 = never, n > 1 = n slices summed by a second pass, -n = a thread-block cluster of n along K; 0 = automatic. */
int odl_debug_set_split_k(int splits);
/* K elements per pipeline stage of the 256-wide tile of the one-CTA kernel: 16 or 32; 0 = automatic. */
int odl_debug_set_bk(int bk);
/* K-slabs per pipeline stage in plain TF32: 1 or 2; 0 = automatic. */
int odl_debug_set_slabs(int n);
/* CTA pairs (cta_group::2): 0 = where it pays, 1 = never, 2 = whenever the shape allows (one tile per pair, never the
 * persistent kernel), 3 = 2-D copies for MN-major
 * operands, 4 = never the 256 x 512 plain-TF32 tile, 5 = like 2 plus that tile for every plain-TF32 problem,
 * 6 = never the persistent kernel, 7 = the persistent kernel whenever the shape allows. */
int odl_debug_set_pair_mode(int mode);
/* CTA pairs the persistent kernel walks its tiles with; 0 = as many as the GPU holds at once.  Small values make small
 * test shapes run several rounds and a split last round.  A negative value -n uses n pairs with the fixed assignment
 * (pair p takes units p, p + n, ...) instead of drawing units from the global counter. */
int odl_debug_set_persistent_pairs(int pairs);
/* Stream-K in the persistent kernel (even K ranges per pair instead of whole tiles): 0 = where it pays (at most half
 * as many tiles as pairs), 1 = always, -1 = never. */
int odl_debug_set_stream_k(int mode);
/* Conv2d: 0 = automatic, 1 = explicit im2col + GEMM everywhere, 2 = implicit-GEMM weight gradient instead of the direct
 * kernel for small layers, 3 = implicit-GEMM forward instead of the direct kernel for small layers, 4 = the generic direct
 * input-gradient kernel also for the shapes that have a compile-time variant, 5 = the compile-time variant with one position
 * per thread where it would take two, 6 = the direct weight-gradient kernel that gathers column blocks also where
 * the one that stages image tiles would run, 7 = the latter wherever its window fits shared memory,
 * 8 = four input channels per thread in the compile-time input-gradient kernels where they would take eight. */
int odl_debug_set_conv_mode(int mode);

/* Number of NVTX ranges the training-step entry points have opened in this process: 0 unless the environment variable
 * ODL_NVTX is set to a non-zero value (lets a test see the switch work without a profiler attached). */
long long odl_debug_nvtx_ranges(void);

/* Device address of the int that kernels raise when a bounded wait runs out (what odl_device_status reads and clears);
 * NULL before odl_init.  For a test kernel that lets such a wait run out on purpose (tests/cuda/). */
int *odl_debug_error_flag(void);

#ifdef __cplusplus
}
#endif
#endif /* ODL_B200_TEST_H_ */

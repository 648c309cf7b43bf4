/*
 * kernl_b200 — test and measurement hooks. NOT part of the stable C ABI: names, arguments and
 * behaviour may change between versions. Every hook sets PROCESS-WIDE state that all later calls
 * of all threads see, so they belong in tests and A/B measurements, not in a serving process.
 * None of them has a counterpart in the reference project.
 */
#ifndef KERNL_B200_DEBUG_H
#define KERNL_B200_DEBUG_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Force the column-tile width of the tcgen05 GEMM (32/64/128/256; 0 = cost model). */
void kb_debug_force_bn(int bn);
/* Force the number of K splits of the GEMM (0 = heuristic; needs a workspace). */
void kb_debug_force_splits(int splits);
/* Query tiles per CTA of the head-dimension-64 attention kernel (0 = dispatcher's choice, 1, 2). */
void kb_debug_split_tiles(int tiles);
/* Work scheduling of the head-dimension-64 attention kernel: 1 = persistent CTAs that pull query
 * tiles from a device-side queue, 2 = the same without the longest-batch-first tile order,
 * 0 = one CTA per query tile, -1 = dispatcher's choice. */
void kb_debug_attention_persistent(int mode);
/* 0 = large GEMMs stay on the one-CTA-per-tile kernel instead of CTA pairs on 256-row tiles;
 * 192 / 256 = CTA pairs with that tile width whatever the cost model says; 1 = dispatcher's choice. */
void kb_debug_linear_pair(int mode);
/* 0 = launch every kernel with plain stream ordering instead of programmatic dependent launch. */
void kb_debug_pdl(int on);
/* Limits (SM clock cycles) of the bounded device-side waits on the CURRENT device: waits inside one
 * kernel, and waits on another rank's flag. A value <= 0 restores that limit's default. Lets a test
 * make a wait give up on purpose: the kernel then records KB_ERR_TIMEOUT in the status word and
 * returns; nothing traps or hangs. Synchronises the device. Returns a KB_* status. */
int kb_debug_wait_limit(int64_t in_kernel_cycles, int64_t peer_cycles);

#ifdef __cplusplus
}
#endif
#endif /* KERNL_B200_DEBUG_H */

// How work is dealt to persistent CTAs, shared by the kernels and the host-side planner.
//
// A "unit" is 256 consecutive k of one weight row (one GGUF super-block, or the codes and group
// parameters of 256 k of an affine pack); a "panel" is a run of consecutive output rows. The
// (panel, unit) pairs are numbered panel-major and cut into equal contiguous runs, one per CTA,
// so every SM streams the same number of bytes whatever N and K are. A panel whose units are
// spread over several CTAs is combined through fp32 scratch slots: every contributor parks its
// partial sums in its own slot and bumps an arrival counter; the last to arrive adds the slots in
// slot order, so the result does not depend on arrival order.
#pragma once
#include "ishi_ptx.cuh"

namespace ishi {

constexpr int kMaxSrc = 4;

// Which CTA owns quantum q when Q quanta are dealt to G CTAs in runs
// [floor(j*Q/G), floor((j+1)*Q/G)).
__host__ __device__ inline long long cta_of_quantum(long long q, long long Q, long long G) {
  return ((q + 1) * G - 1) / Q;
}

// How many CTAs contribute to panel p (each panel has `units` quanta, there are P panels and G
// CTAs), and the first of them. With fewer quanta than CTAs every CTA holds at most one quantum,
// so a panel's contributors are its quanta (first = -1: the slot is the unit index); otherwise
// every CTA between the owners of the panel's first and last quantum holds part of it.
__host__ __device__ inline int panel_touch(int p, int units, int P, int G, long long *first) {
  const long long Q = (long long)P * units;
  if (Q < G) {
    if (first) *first = -1;
    return units;
  }
  const long long jf = cta_of_quantum((long long)p * units, Q, G);
  const long long jl = cta_of_quantum((long long)(p + 1) * units - 1, Q, G);
  if (first) *first = jf;
  return (int)(jl - jf + 1);
}

}  // namespace ishi

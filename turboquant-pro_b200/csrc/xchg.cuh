// Device-side view of a peer-memory exchange (see xchg.cu) and the steps of one exchange, shared
// by the stand-alone exchange kernel and by the merge kernel of the tensor-core decode, which
// can publish and merge its rows itself.
#pragma once
#include "common.cuh"

constexpr int TQ_XCHG_MAX_WORLD = 16;  // most ranks

struct XchgDev {
  float* peer[TQ_XCHG_MAX_WORLD];  // every rank's region (own included)
  int rank, world, rows, phases;
  size_t flags_off, ctrl_off;      // byte offsets inside a region
  unsigned spin_limit;
};

struct tq_xchg {
  int device, rank, world, rows, n_cta;
  size_t bytes, flags_off, ctrl_off;
  float* own;
  float* peer[TQ_XCHG_MAX_WORLD];
  bool ipc[TQ_XCHG_MAX_WORLD];
  unsigned spin_limit;
};

// fills the kernel-side view; false if a peer is not connected yet
bool tq_xchg_view(const tq_xchg* x, int phases, XchgDev* out);

#ifdef __CUDACC__
TQ_DEV unsigned xchg_ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
TQ_DEV void xchg_st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
TQ_DEV unsigned* xchg_ctrl(const XchgDev& x) {
  return (unsigned*)((uint8_t*)x.peer[x.rank] + x.ctrl_off);
}
// number of the exchange under way (the last finished one + 1)
TQ_DEV unsigned xchg_epoch(const XchgDev& x) { return *(volatile unsigned*)&xchg_ctrl(x)[0] + 1u; }
// where rank `src`'s state of `row` lives in rank `dst`'s region
TQ_DEV float* xchg_row(const XchgDev& x, int dst, int slot, int src, int row) {
  return x.peer[dst] + (((size_t)slot * x.world + src) * x.rows + row) * TQ_PART_STRIDE;
}
// flag of row `idx` of rank `src` in rank `dst`'s region
TQ_DEV unsigned* xchg_flag(const XchgDev& x, int dst, int slot, int src, int idx) {
  return (unsigned*)((uint8_t*)x.peer[dst] + x.flags_off) + ((size_t)slot * x.world + src) * x.rows + idx;
}
// Thread e < world tells rank e that this rank's row `idx` of exchange `ep` is written.
// Call after a CTA barrier that follows the row stores: the release store orders them, as
// this thread's predecessors, before the flag at system scope.
TQ_DEV void xchg_signal(const XchgDev& x, int e, int slot, int idx, unsigned ep) {
  if (e < x.world) xchg_st_release_sys(xchg_flag(x, e, slot, x.rank, idx), ep);
}
// Thread e < world waits (bounded) for rank e's row `idx`; returns false where the wait
// ran out (bit 0 of the status word is then set).  Follow with a CTA barrier.
TQ_DEV bool xchg_wait(const XchgDev& x, int e, int slot, int idx, unsigned ep) {
  if (e >= x.world) return true;
  const unsigned* flag = xchg_flag(x, x.rank, slot, e, idx);
  unsigned n = 0;
  // (flags only grow; the signed difference keeps the test right across a wrap)
  while ((int)(xchg_ld_acquire_sys(flag) - ep) < 0) {
    if (++n >= x.spin_limit) {
      atomicOr(&xchg_ctrl(x)[2], 1u);
      return false;
    }
    __nanosleep(32);
  }
  return true;
}
// Element e of the merged output of `row`: the states of all ranks in rank order, the
// arithmetic of merge_partials (kv_fused.py:139-153) as in lse_combine_kernel.  Read past the
// first-level cache: the rows were written by other GPUs.
TQ_DEV float xchg_merge_row(const XchgDev& x, int slot, int row, int e) {
  float M = -INFINITY;
  for (int p = 0; p < x.world; ++p) M = fmaxf(M, __ldcg(&xchg_row(x, x.rank, slot, p, row)[0]));
  float L = 0.0f, A = 0.0f;
  for (int p = 0; p < x.world; ++p) {
    const float* r = xchg_row(x, x.rank, slot, p, row);
    const float m = __ldcg(&r[0]);
    const float w = m > -INFINITY ? __expf(m - M) : 0.0f;
    L += __ldcg(&r[1]) * w;
    A += __ldcg(&r[2 + e]) * w;
  }
  return L > 0.0f ? A / L : 0.0f;
}
// The last of `n_cta` CTAs to get here closes exchange `ep` (thread 0 of each CTA calls this
// after a CTA barrier).
TQ_DEV void xchg_close(const XchgDev& x, unsigned n_cta, unsigned ep) {
  unsigned* ctrl = xchg_ctrl(x);
  __threadfence();
  const unsigned prev = atomicAdd(&ctrl[1], 1u);
  if (prev == n_cta - 1u) {
    ctrl[1] = 0u;
    *(volatile unsigned*)&ctrl[0] = ep;
  }
}
#endif

// Exchange of the per-rank attention states (m, l, o[D]) of a sequence split over several
// GPUs, fused with their log-sum-exp merge: one kernel per decode step and layer instead of a
// library all-gather followed by a merge kernel.
//
// Every rank owns one region of device memory with the same layout and maps the regions of
// the other ranks (CUDA IPC between processes, plain pointers inside one process):
//
//   gather  [2 slots][world][rows][2 + D] float32   the states as written by their owners
//   flags   [2 slots][world][rows] uint32           "rank r has written row i of exchange e"
//   ctrl    epoch, CTA counter, status
//
// Exchange number e (1, 2, ...) uses slot e & 1.  CTA c of a rank owns rows c, c + n_cta, ...
// (the merge kernel of the tensor-core decode, which can run the exchange itself, owns the rows
// of its unit); flags are per row, so the two forms can be mixed:
// it stores its rows of the local states into slot e & 1 of every rank's gather area with
// plain peer stores over NVLink and writes e into the rows' flags on every rank with a
// system-scope release store; then it waits until the flags of its rows from all ranks show e
// in its own region and merges the rows in rank order (the arithmetic of merge_partials, kv_fused.py:139-153, as in
// lse_combine_kernel).  A CTA depends only on the rows it merges, so nothing waits on a whole
// grid.  Two slots suffice: a rank can start exchange e + 1 only after its
// own exchange e is complete, which needed every other rank's flag for e, which that rank
// wrote after its exchange e - 1 had completed (stream order), so nobody still reads the slot
// that exchange e + 1 overwrites.
//
// The wait is bounded: after `spin_limit` probes the kernel sets bit 0 of the status word,
// writes zeros for the rows it could not merge and returns.  No multicast, no multimem: plain
// loads and stores on peer memory.
#include <cstring>

#include "xchg.cuh"

namespace {

constexpr int TQ_XCHG_CTAS = 32;             // most CTAs (row groups) of the exchange kernel
constexpr unsigned TQ_XCHG_SPIN = 1u << 22;  // default probes per wait (each takes 0.1 us or more)

struct XchgArgs {
  XchgDev x;
  int n_cta;
  const float* mlo;  // [rows][2 + D] local states
  float* out;        // [rows][D]
};

__global__ void __launch_bounds__(TQ_D) xchg_kernel(XchgArgs a) {
  const int e = threadIdx.x, c = blockIdx.x;
  const XchgDev& x = a.x;
  // launched as a programmatic dependent: scheduled while the kernel before it in the stream
  // (the one that writes the local states) drains, it waits for that kernel here and lets
  // the kernel after it be scheduled in turn
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const unsigned ep = xchg_epoch(x);
  const int slot = (int)(ep & 1u);

  if (x.phases & 1) {
    for (int row = c; row < x.rows; row += a.n_cta) {
      const float* src = a.mlo + (size_t)row * TQ_PART_STRIDE;
      const float v0 = src[e];
      const float v1 = e < 2 ? src[TQ_D + e] : 0.0f;
      for (int p = 0; p < x.world; ++p) {
        float* dst = xchg_row(x, p, slot, x.rank, row);
        dst[e] = v0;
        if (e < 2) dst[TQ_D + e] = v1;
      }
    }
    __syncthreads();
    for (int row = c; row < x.rows; row += a.n_cta) xchg_signal(x, e, slot, row, ep);
  }
  if (x.phases & 2) {
    __shared__ int s_fail;
    if (e == 0) s_fail = 0;
    __syncthreads();
    for (int row = c; row < x.rows; row += a.n_cta)
      if (!xchg_wait(x, e, slot, row, ep)) {
        s_fail = 1;
        break;
      }
    __syncthreads();
    const bool fail = s_fail != 0;
    for (int row = c; row < x.rows; row += a.n_cta)
      a.out[(size_t)row * TQ_D + e] = fail ? 0.0f : xchg_merge_row(x, slot, row, e);
    __syncthreads();
    if (e == 0) xchg_close(x, (unsigned)a.n_cta, ep);
  }
}

}  // namespace

bool tq_xchg_view(const tq_xchg* x, int phases, XchgDev* out) {
  for (int p = 0; p < TQ_XCHG_MAX_WORLD; ++p) {
    out->peer[p] = p < x->world ? x->peer[p] : nullptr;
    if (p < x->world && x->peer[p] == nullptr) return false;
  }
  out->rank = x->rank;
  out->world = x->world;
  out->rows = x->rows;
  out->phases = phases;
  out->flags_off = x->flags_off;
  out->ctrl_off = x->ctrl_off;
  out->spin_limit = x->spin_limit;
  return true;
}

extern "C" {

int32_t tq_xchg_create(int32_t device, int32_t rank, int32_t world, int32_t rows, int32_t head_dim,
                       tq_xchg** out) {
  TQ_REQUIRE(out != nullptr, TQ_ERR_INVALID, "null argument");
  TQ_REQUIRE(head_dim == TQ_D, TQ_ERR_UNSUPPORTED, "only head_dim == 128 is implemented");
  TQ_REQUIRE(world >= 1 && world <= TQ_XCHG_MAX_WORLD && rank >= 0 && rank < world, TQ_ERR_INVALID,
             "bad rank / world (at most 16 ranks)");
  TQ_REQUIRE(rows >= 1, TQ_ERR_INVALID, "rows must be positive");
  TQ_CUDA(cudaSetDevice(device));
  tq_xchg* x = new tq_xchg();
  x->device = device;
  x->rank = rank;
  x->world = world;
  x->rows = rows;
  x->n_cta = rows < TQ_XCHG_CTAS ? rows : TQ_XCHG_CTAS;
  x->flags_off = align_up((size_t)2 * world * rows * TQ_PART_STRIDE * sizeof(float), 256);
  x->ctrl_off = x->flags_off + align_up((size_t)2 * world * rows * sizeof(unsigned), 256);
  x->bytes = x->ctrl_off + 256;
  x->spin_limit = TQ_XCHG_SPIN;
  for (int p = 0; p < TQ_XCHG_MAX_WORLD; ++p) {
    x->peer[p] = nullptr;
    x->ipc[p] = false;
  }
  cudaError_t e = cudaMalloc((void**)&x->own, x->bytes);
  if (e == cudaSuccess) e = cudaMemset(x->own, 0, x->bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    delete x;
    return tq_cuda_fail(e, "allocating the exchange region");
  }
  x->peer[rank] = x->own;
  *out = x;
  return TQ_OK;
}

int32_t tq_xchg_destroy(tq_xchg* x) {
  if (x == nullptr) return TQ_OK;
  cudaSetDevice(x->device);
  for (int p = 0; p < x->world; ++p)
    if (x->ipc[p] && x->peer[p] != nullptr) cudaIpcCloseMemHandle(x->peer[p]);
  cudaFree(x->own);
  delete x;
  return TQ_OK;
}

int64_t tq_xchg_region_bytes(const tq_xchg* x) { return x ? (int64_t)x->bytes : 0; }

void* tq_xchg_base(const tq_xchg* x) { return x ? (void*)x->own : nullptr; }

int32_t tq_xchg_ipc_handle(tq_xchg* x, void* handle64) {
  TQ_REQUIRE(x != nullptr && handle64 != nullptr, TQ_ERR_INVALID, "null argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  TQ_CUDA(cudaSetDevice(x->device));
  cudaIpcMemHandle_t h;
  TQ_CUDA(cudaIpcGetMemHandle(&h, x->own));
  std::memcpy(handle64, &h, sizeof(h));
  return TQ_OK;
}

int32_t tq_xchg_open_peer(tq_xchg* x, int32_t peer_rank, const void* handle64) {
  TQ_REQUIRE(x != nullptr && handle64 != nullptr, TQ_ERR_INVALID, "null argument");
  TQ_REQUIRE(peer_rank >= 0 && peer_rank < x->world && peer_rank != x->rank, TQ_ERR_INVALID,
             "bad peer rank");
  TQ_REQUIRE(x->peer[peer_rank] == nullptr, TQ_ERR_INVALID, "peer already connected");
  TQ_CUDA(cudaSetDevice(x->device));
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  TQ_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  x->peer[peer_rank] = (float*)p;
  x->ipc[peer_rank] = true;
  return TQ_OK;
}

int32_t tq_xchg_set_peer(tq_xchg* x, int32_t peer_rank, void* region) {
  TQ_REQUIRE(x != nullptr && region != nullptr, TQ_ERR_INVALID, "null argument");
  TQ_REQUIRE(peer_rank >= 0 && peer_rank < x->world && peer_rank != x->rank, TQ_ERR_INVALID,
             "bad peer rank");
  x->peer[peer_rank] = (float*)region;
  x->ipc[peer_rank] = false;
  return TQ_OK;
}

int32_t tq_xchg_set_wait_limit(tq_xchg* x, int32_t probes) {
  TQ_REQUIRE(x != nullptr, TQ_ERR_INVALID, "null argument");
  x->spin_limit = probes > 0 ? (unsigned)probes : TQ_XCHG_SPIN;
  return TQ_OK;
}

int32_t tq_xchg_gather_merge(tq_xchg* x, const float* mlo, float* out, int32_t phases,
                             void* stream) {
  TQ_REQUIRE(x != nullptr && mlo != nullptr, TQ_ERR_INVALID, "null argument");
  TQ_REQUIRE(phases >= 1 && phases <= 3, TQ_ERR_INVALID, "phases: 1 publish, 2 wait and merge, 3 both");
  TQ_REQUIRE(out != nullptr || !(phases & 2), TQ_ERR_INVALID, "out must be a device pointer");
  XchgArgs a;
  TQ_REQUIRE(tq_xchg_view(x, phases, &a.x), TQ_ERR_INVALID, "a peer region is not connected");
  TQ_CUDA(cudaSetDevice(x->device));
  a.n_cta = x->n_cta;
  a.mlo = mlo;
  a.out = out;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(x->n_cta);
  cfg.blockDim = dim3(TQ_D);
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  TQ_CUDA(cudaLaunchKernelEx(&cfg, xchg_kernel, a));
  return TQ_OK;
}

int32_t tq_xchg_status(tq_xchg* x, int32_t* status, void* stream) {
  TQ_REQUIRE(x != nullptr && status != nullptr, TQ_ERR_INVALID, "null argument");
  TQ_CUDA(cudaSetDevice(x->device));
  unsigned v = 0;
  TQ_CUDA(cudaMemcpyAsync(&v, (uint8_t*)x->own + x->ctrl_off + 8, 4, cudaMemcpyDeviceToHost,
                          (cudaStream_t)stream));
  TQ_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  *status = (int32_t)v;
  return TQ_OK;
}

}  // extern "C"

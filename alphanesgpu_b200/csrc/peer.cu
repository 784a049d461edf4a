// Gradient exchange of data-parallel training over NVLink peer memory, fused with the optimiser update.
//
// What hvd.DistributedOptimizer does variable by variable in the reference (STAF/staf_train.py:484-487: average
// the gradients over the ranks, then Adam) as ONE kernel per rank and step, with one NVLink trip on its critical
// path.  Every rank owns a receive area that the other ranks of the node have mapped (CUDA IPC): one 8-byte word
// per (source rank, element) holding the element's bits and the number of the step it belongs to.  The kernel
//   1. stores its own gradient, element by element, into its slot of every peer's receive area (8-byte
//      system-scope stores: value and step tag arrive together, so no flag, no fence and no second trip is needed),
//   2. polls its own receive area until every peer's element carries this step's tag (bounded in time),
//   3. agrees over the whole grid whether everything arrived - one decision per launch: either every block
//      applies the update or none does; a launch that gives up records STAFB_ERR_PEER_TIMEOUT and leaves theta,
//      the moments and the step counter untouched -,
//   4. sums the gradients in rank order (every rank computes bit-identical sums, the replicas of theta never
//      drift), divides by the world size and applies Adam.
// A rank that gave up and a late rank that then went ahead hold different parameters from that step on: the
// host has to notice the status and re-broadcast (alphanesgpu_b200/train.py does, at every collection point).
// Two receive areas alternate from step to step: a fast peer that already stores step k+1 does not touch what
// this rank still reads for step k, and no rank can run two steps ahead of another because step k+1 cannot
// complete without every peer's elements of step k+1.  There is no multicast object, no collective library and
// no second launch between the backward pass and the parameter update.
#include <math.h>
#include <string.h>

#include "common.cuh"

namespace stafb {

constexpr int PEER_MAX = 16;
constexpr int PEER_PUSH = 1, PEER_CONSUME = 2;  // phases of the kernel (both in one launch unless ranks share a GPU)

struct PeerView {
  int rank, world;
  const void* grad;                       // this rank's gradient of this launch's parity
  const unsigned long long* recv;         // own receive area of that parity: [PEER_MAX][words per rank]
  unsigned long long* recv_of[PEER_MAX];  // the peers' receive areas of that parity
};

__device__ __forceinline__ unsigned long long ld_sys64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_sys64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// an element as tagged 8-byte words: one for fp32 (bits | tag << 32), two for fp64 (low half, high half)
template <class T> struct PeerWords;
template <> struct PeerWords<float> {
  static constexpr int W = 1;
  static __device__ __forceinline__ void push(unsigned long long* dst, float x, unsigned tag) {
    st_sys64(dst, ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(x));
  }
  static __device__ __forceinline__ bool poll(const unsigned long long* src, unsigned tag, float& x) {
    const unsigned long long w = ld_sys64(src);
    x = __uint_as_float((unsigned)w);
    return (unsigned)(w >> 32) == tag;
  }
};
template <> struct PeerWords<double> {
  static constexpr int W = 2;
  static __device__ __forceinline__ void push(unsigned long long* dst, double x, unsigned tag) {
    const unsigned long long b = (unsigned long long)__double_as_longlong(x);
    st_sys64(dst, ((unsigned long long)tag << 32) | (b & 0xFFFFFFFFull));
    st_sys64(dst + 1, ((unsigned long long)tag << 32) | (b >> 32));
  }
  static __device__ __forceinline__ bool poll(const unsigned long long* src, unsigned tag, double& x) {
    const unsigned long long lo = ld_sys64(src), hi = ld_sys64(src + 1);
    x = __longlong_as_double((long long)((hi << 32) | (lo & 0xFFFFFFFFull)));
    return (unsigned)(lo >> 32) == tag && (unsigned)(hi >> 32) == tag;
  }
};

// status: [0] first error, [1] unused, [2] blocks that saw everything, [3] blocks that gave up (both cleared by the
// block that finishes last).  step_d: [0] updates applied so far, [1] blocks done.  The grid must be resident as
// a whole (256-thread blocks, at most eight per SM: up to ~300,000 parameters), because its blocks wait for each
// other's finding.
template <class T>
__global__ void __launch_bounds__(256)
    k_allreduce_adam(PeerView pv, int n, T* __restrict__ theta, T* __restrict__ m, T* __restrict__ v, double lr,
                     double b1, double b2, T eps, int* __restrict__ step_d, long long wait_cycles,
                     int* __restrict__ status, int phase) {
  __shared__ int ok_s;
  typedef PeerWords<T> PW;
  chain_wait();  // the gradient is the output of the kernel before this one
  const int step = *reinterpret_cast<volatile int*>(step_d) + 1;  // the update being applied; equal on all ranks
  const unsigned tag = (unsigned)step;
  const int q = blockIdx.x * blockDim.x + threadIdx.x;
  const size_t per_rank = (size_t)n * PW::W;
  T g_own = T(0);
  if (q < n) g_own = reinterpret_cast<const T*>(pv.grad)[q];
  if ((phase & PEER_PUSH) && q < n) {
    // first of all: the peers are waiting for it
#pragma unroll
    for (int r = 0; r < PEER_MAX; r++)
      if (r < pv.world && r != pv.rank) PW::push(pv.recv_of[r] + (size_t)pv.rank * per_rank + (size_t)q * PW::W, g_own, tag);
  }
  if (!(phase & PEER_CONSUME)) return;
  // everything that does not need the peers while their stores are on the way
  T m_old = T(0), v_old = T(0), th_old = T(0);
  if (q < n) { m_old = m[q]; v_old = v[q]; th_old = theta[q]; }
  const T lr_t = (T)(lr * sqrt(1.0 - pow(b2, (double)step)) / (1.0 - pow(b1, (double)step)));
  T gv[PEER_MAX];
  unsigned pending = 0u;
  if (q < n)
    for (int r = 0; r < pv.world; r++)
      if (r != pv.rank) pending |= 1u << r;
  const long long t0 = clock64();
  while (pending) {
    // all outstanding peers in one round: their loads are in flight together
#pragma unroll
    for (int r = 0; r < PEER_MAX; r++)
      if ((pending >> r) & 1u) {
        T x;
        if (PW::poll(pv.recv + (size_t)r * per_rank + (size_t)q * PW::W, tag, x)) { gv[r] = x; pending &= ~(1u << r); }
      }
    if (pending) {
      const long long waited = clock64() - t0;
      if (waited > wait_cycles) break;
      if (waited > 20000) __nanosleep(100);  // spin for the first ~10 us, then back off
    }
  }
  // one decision per launch: every block reports what it found, then reads the tally once it is complete
  const int blk_ok = __syncthreads_and(pending == 0u);
  if (threadIdx.x == 0) {
    atomicAdd(status + (blk_ok ? 2 : 3), 1);
    int ok = 0;
    const long long t1 = clock64();
    while (true) {
      const int a = *reinterpret_cast<volatile int*>(status + 2), f = *reinterpret_cast<volatile int*>(status + 3);
      if (a + f >= (int)gridDim.x) { ok = f == 0; break; }
      if (clock64() - t1 > wait_cycles + 4000000000ll) break;  // a block that never ran: the grid was too large
    }
    if (!ok) atomicCAS(status, 0, STAFB_ERR_PEER_TIMEOUT);
    ok_s = ok;
  }
  __syncthreads();
  const int ok = ok_s;
  if (ok && q < n) {
    // the sum is taken in rank order, so every rank computes the same bits
    T g = T(0);
#pragma unroll
    for (int r = 0; r < PEER_MAX; r++)
      if (r < pv.world) g += (r == pv.rank) ? g_own : gv[r];
    g *= T(1) / T(pv.world);
    const T mm = (T)b1 * m_old + (T(1) - (T)b1) * g;
    const T vv = (T)b2 * v_old + (T(1) - (T)b2) * g * g;
    m[q] = mm;
    v[q] = vv;
    theta[q] = th_old - lr_t * mm / (r_sqrt(vv) + eps);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(step_d + 1, 1) == (int)gridDim.x - 1) {
      // every block has read the tally by now: cleared for the next launch.  A launch that gave up leaves
      // theta, m, v AND the step count as they were, so that a repeated launch decides anew.
      step_d[1] = 0;
      status[2] = 0;
      status[3] = 0;
      __threadfence();
      if (ok) atomicAdd(step_d, 1);
    }
  }
}

}  // namespace stafb

using namespace stafb;

// One rank's side of the exchange.  Block layout (device memory of this rank, mapped by the peers):
//   [ grad parity 0 : n elements | grad parity 1 : n elements | recv[2][PEER_MAX][n elements as tagged words] ]
struct stafb_peer {
  int rank, world, n, dtype;
  size_t es, grad_bytes, recv_words;  // recv_words: 8-byte words of one source rank's slot
  char* block;             // own allocation
  char* peer[PEER_MAX];    // mapped blocks (own rank: block)
  int connected;
  int* status_d;
  long long wait_cycles;
};

extern "C" int stafb_peer_create(stafb_ctx* c, int rank, int world, int n_params, stafb_peer** out) {
  if (!c || !out || world < 1 || world > PEER_MAX || rank < 0 || rank >= world || n_params <= 0)
    return STAFB_ERR_INVALID;
  stafb_peer* p = (stafb_peer*)calloc(1, sizeof(stafb_peer));
  if (!p) return STAFB_ERR_INVALID;
  p->rank = rank; p->world = world; p->n = n_params; p->dtype = c->dtype;
  p->es = c->dtype == STAFB_F32 ? 4 : 8;
  p->grad_bytes = ((p->es * (size_t)n_params + 255) / 256) * 256;
  p->recv_words = (size_t)n_params * (p->es / 4);
  const size_t bytes = 2 * p->grad_bytes + 2 * (size_t)PEER_MAX * p->recv_words * sizeof(unsigned long long);
  STAFB_CUDA_OK(cudaMalloc((void**)&p->block, bytes));
  STAFB_CUDA_OK(cudaMemset(p->block, 0, bytes));
  STAFB_CUDA_OK(cudaMalloc((void**)&p->status_d, 4 * sizeof(int)));  // status word, spare, the launch's tally
  STAFB_CUDA_OK(cudaMemset(p->status_d, 0, 4 * sizeof(int)));
  STAFB_CUDA_OK(cudaDeviceSynchronize());
  p->peer[rank] = p->block;
  int khz = 1500000;
  cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, c->device);
  p->wait_cycles = 2LL * khz * 1000;  // about two seconds of SM clock
  if (getenv("STAFB_PEER_WAIT_MS")) p->wait_cycles = (long long)atoll(getenv("STAFB_PEER_WAIT_MS")) * khz;
  p->connected = world == 1;
  *out = p;
  return STAFB_OK;
}

extern "C" int stafb_peer_handle(stafb_peer* p, void* handle64) {
  if (!p || !handle64) return STAFB_ERR_INVALID;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  cudaIpcMemHandle_t h;
  STAFB_CUDA_OK(cudaIpcGetMemHandle(&h, p->block));
  memcpy(handle64, &h, 64);
  return STAFB_OK;
}

extern "C" int stafb_peer_connect(stafb_peer* p, const void* handles) {
  if (!p || !handles) return STAFB_ERR_INVALID;
  for (int r = 0; r < p->world; r++) {
    if (r == p->rank || p->peer[r]) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, (const char*)handles + 64 * (size_t)r, 64);
    void* ptr = nullptr;
    STAFB_CUDA_OK(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
    p->peer[r] = (char*)ptr;
  }
  p->connected = 1;
  return STAFB_OK;
}

// Ranks that live in ONE process (one thread or stream per GPU, or several emulated ranks on one GPU in a test)
// connect through their handles directly, without IPC.
extern "C" int stafb_peer_connect_local(stafb_peer* p, stafb_peer* const* all) {
  if (!p || !all) return STAFB_ERR_INVALID;
  for (int r = 0; r < p->world; r++) {
    if (r == p->rank) continue;
    if (!all[r] || all[r]->world != p->world || all[r]->rank != r || all[r]->n != p->n) return STAFB_ERR_INVALID;
    p->peer[r] = all[r]->block;
  }
  p->connected = 2;  // nothing to unmap on destroy
  return STAFB_OK;
}

extern "C" int stafb_peer_set_wait_ms(stafb_peer* p, long long ms) {
  if (!p || ms < 0) return STAFB_ERR_INVALID;
  int dev = 0, khz = 1500000;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev);
  p->wait_cycles = ms * (long long)khz;
  return STAFB_OK;
}

extern "C" void* stafb_peer_grad(stafb_peer* p, int parity) {
  if (!p || parity < 0 || parity > 1) return nullptr;
  return p->block + (size_t)parity * p->grad_bytes;
}

extern "C" int stafb_peer_status(stafb_peer* p) {
  if (!p) return STAFB_ERR_INVALID;
  int s = 0;
  STAFB_CUDA_OK(cudaMemcpy(&s, p->status_d, sizeof(int), cudaMemcpyDeviceToHost));
  return s;
}

extern "C" void stafb_peer_destroy(stafb_peer* p) {
  if (!p) return;
  for (int r = 0; r < p->world && p->connected == 1; r++)
    if (r != p->rank && p->peer[r]) cudaIpcCloseMemHandle(p->peer[r]);
  cudaFree(p->block);
  cudaFree(p->status_d);
  free(p);
}

// phase: PEER_PUSH | PEER_CONSUME in one launch (ranks on GPUs of their own), or the two as separate launches for
// ranks that share ONE GPU (tests): all ranks' pushes first, then their consumes - kernels on one GPU must never
// wait for one another.
extern "C" int stafb_allreduce_adam_phase(stafb_ctx* c, stafb_peer* p, void* stream, int parity, void* theta, void* mm,
                                          void* vv, double lr, double b1, double b2, double eps, int* step_d,
                                          int phase) {
  if (!c || !p || !theta || !mm || !vv || !step_d || parity < 0 || parity > 1 || !p->connected || phase < 1 ||
      phase > 3)
    return STAFB_ERR_INVALID;
  if (c->dtype != p->dtype) return STAFB_ERR_INVALID;
  const int n = p->n, grid = (n + 255) / 256;
  int nsm = 148;
  cudaDeviceGetAttribute(&nsm, cudaDevAttrMultiProcessorCount, c->device);
  if (grid > 8 * nsm) return STAFB_ERR_CAPACITY;  // the blocks wait for each other: the grid must be resident
  PeerView pv;
  memset(&pv, 0, sizeof(pv));
  pv.rank = p->rank;
  pv.world = p->world;
  pv.grad = p->block + (size_t)parity * p->grad_bytes;
  const size_t area = (size_t)PEER_MAX * p->recv_words;  // words of one parity's receive area
  for (int r = 0; r < p->world; r++)
    pv.recv_of[r] = reinterpret_cast<unsigned long long*>(p->peer[r] + 2 * p->grad_bytes) + (size_t)parity * area;
  pv.recv = pv.recv_of[p->rank];
  cudaStream_t s = (cudaStream_t)stream;
  if (c->dtype == STAFB_F32)
    STAFB_CUDA_OK(launch_chained(k_allreduce_adam<float>, grid, 256, 0, s, pv, n, (float*)theta, (float*)mm,
                                 (float*)vv, lr, b1, b2, (float)eps, step_d, p->wait_cycles, p->status_d, phase));
  else
    STAFB_CUDA_OK(launch_chained(k_allreduce_adam<double>, grid, 256, 0, s, pv, n, (double*)theta, (double*)mm,
                                 (double*)vv, lr, b1, b2, eps, step_d, p->wait_cycles, p->status_d, phase));
  return STAFB_OK;
}

extern "C" int stafb_allreduce_adam(stafb_ctx* c, stafb_peer* p, void* stream, int parity, void* theta, void* mm,
                                    void* vv, double lr, double b1, double b2, double eps, int* step_d) {
  return stafb_allreduce_adam_phase(c, p, stream, parity, theta, mm, vv, lr, b1, b2, eps, step_d,
                                    PEER_PUSH | PEER_CONSUME);
}

// Gradient exchange of data-parallel training over NVLink peer memory, fused with the optimiser update.
//
// What hvd.DistributedOptimizer does variable by variable in the reference (STAF/staf_train.py:484-487: average
// the gradients over the ranks, then Adam) as ONE kernel per rank and step.  Every rank accumulates its gradient
// in a buffer of its own device memory that the other ranks of the node have mapped (CUDA IPC).  The kernel
//   1. publishes "my gradient of this step is complete" in a flag word on every peer (a system-scope store
//      over NVLink after a system fence),
//   2. waits until all peers have published theirs (polling flag words in its OWN memory; bounded in time -
//      when the bound is hit the launch as a whole records STAFB_ERR_PEER_TIMEOUT, leaves theta, the moments and
//      the step counter untouched and returns: the decision is taken once per launch, see the kernel),
//   3. reads the peers' gradients with plain peer loads, all in flight together, sums them in rank order (so
//      that every rank computes bit-identical sums and the replicas of theta never drift), divides by the world
//      size and applies Adam.
// A rank that gave up and a late rank that then went ahead hold different parameters from that step on: the
// host has to notice the status and re-broadcast (alphanesgpu_b200/train.py does, at every collection point).
// Two gradient buffers alternate from step to step: a rank that is already accumulating step k+1 does not
// touch what a slower peer still reads for step k, and no rank can run two steps ahead of another because step
// k+1 cannot complete without every peer's flag of step k+1.  There is no multicast object, no collective
// library and no second launch between the backward pass and the parameter update.
#include <math.h>
#include <string.h>

#include "common.cuh"

namespace stafb {

constexpr int PEER_MAX = 16;

struct PeerView {
  int rank, world;
  const void* grad[PEER_MAX];  // gradient buffer of every rank for the parity of this launch (own: local pointer)
  int* flag_out[PEER_MAX];     // on rank r: the word this rank writes (flags[parity][my rank] in r's block)
  const int* flag_in;          // own block: flags[parity][0..world)
};

__device__ __forceinline__ int ld_sys(const int* p) {
  int v;
  asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_sys(int* p, int v) {
  asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float ld_peer(const float* p) {
  float v;
  asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ double ld_peer(const double* p) {
  double v;
  asm volatile("ld.relaxed.sys.global.f64 %0, [%1];" : "=d"(v) : "l"(p) : "memory");
  return v;
}

// One decision per launch.  Every block's thread 0 polls the peers' flags (bounded), then proposes its finding
// (all flags seen / gave up) for this step in a verdict word of this rank's own memory with a compare-and-swap;
// the first proposal stands and every block - whenever it runs - adopts it.  So either all blocks apply the
// update or none does, also when a peer's flag lands just as the bound runs out, and the step counter advances
// only with an applied update.  verdict = 2*step + ok; steps only grow, so the word never needs clearing.
template <class T>
__global__ void __launch_bounds__(256)
    k_allreduce_adam(PeerView pv, int n, T* __restrict__ theta, T* __restrict__ m, T* __restrict__ v, double lr,
                     double b1, double b2, T eps, int* __restrict__ step_d /*[2]: step, blocks done*/,
                     long long wait_cycles, int* __restrict__ status /*[2]: status, verdict*/) {
  __shared__ int ok_s;
  chain_wait();  // the gradient is the output of the kernel before this one
  const int step = *reinterpret_cast<volatile int*>(step_d) + 1;  // the update being applied; equal on all ranks
  // everything that does not need the peers is done while thread 0 waits for them: this rank's own values and
  // the step's learning-rate factor (two double-precision powers)
  const int q = blockIdx.x * blockDim.x + threadIdx.x;
  T g_own = T(0), m_old = T(0), v_old = T(0), th_old = T(0);
  if (q < n && threadIdx.x != 0) {
    g_own = reinterpret_cast<const T*>(pv.grad[pv.rank])[q];
    m_old = m[q]; v_old = v[q]; th_old = theta[q];
  }
  const T lr_t = (T)(lr * sqrt(1.0 - pow(b2, (double)step)) / (1.0 - pow(b1, (double)step)));
  if (threadIdx.x == 0) {
    if (blockIdx.x == 0) {
      __threadfence_system();  // this rank's gradient (complete at the kernel boundary) before the flags
      for (int r = 0; r < pv.world; r++)
        if (r != pv.rank) st_sys(pv.flag_out[r], step);
    }
    int seen = 1;
    const long long t0 = clock64();
    for (int r = 0; r < pv.world && seen; r++) {
      if (r == pv.rank) continue;
      while (ld_sys(pv.flag_in + r) < step) {  // flags only grow: a peer is never more than one step ahead
        const long long waited = clock64() - t0;
        if (waited > wait_cycles) { seen = 0; break; }
        if (waited > 20000) __nanosleep(100);  // spin for the first ~10 us, then back off
      }
    }
    int* verdict = status + 1;
    const int want = 2 * step + seen;
    int cur = *reinterpret_cast<volatile int*>(verdict);
    while ((cur >> 1) < step) {
      const int prev = atomicCAS(verdict, cur, want);
      if (prev == cur) { cur = want; break; }
      cur = prev;
    }
    const int ok = ((cur >> 1) == step) ? (cur & 1) : 0;
    if (!ok) atomicCAS(status, 0, STAFB_ERR_PEER_TIMEOUT);
    __threadfence_system();
    ok_s = ok;
  }
  __syncthreads();
  const int ok = ok_s;
  if (q < n && threadIdx.x == 0) {  // thread 0 was busy with the flags
    g_own = reinterpret_cast<const T*>(pv.grad[pv.rank])[q];
    m_old = m[q]; v_old = v[q]; th_old = theta[q];
  }
  if (ok && q < n) {
    // all peers' loads are issued before the first add (one NVLink round trip, not one per rank); the sum is
    // taken in rank order, so every rank computes the same bits
    T gv[PEER_MAX];
#pragma unroll
    for (int r = 0; r < PEER_MAX; r++) {
      gv[r] = T(0);
      if (r < pv.world) {
        const T* gr = reinterpret_cast<const T*>(pv.grad[r]);
        gv[r] = (r == pv.rank) ? g_own : ld_peer(gr + q);
      }
    }
    T g = T(0);
#pragma unroll
    for (int r = 0; r < PEER_MAX; r++)
      if (r < pv.world) g += gv[r];
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
      step_d[1] = 0;
      __threadfence();
      // a launch that gave up leaves theta, m, v AND the step count as they were; every block has read the
      // verdict by now, so it is rewound to "nothing decided for this step" and a repeated launch decides anew
      if (ok) atomicAdd(step_d, 1);
      else status[1] = 2 * step - 1;
    }
  }
}

}  // namespace stafb

using namespace stafb;

// One rank's side of the exchange.  Block layout (device memory of this rank, mapped by the peers):
//   [ grad parity 0 : n elements | grad parity 1 : n elements | flags[2][PEER_MAX] int ]
struct stafb_peer {
  int rank, world, n, dtype;
  size_t es, grad_bytes;
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
  const size_t bytes = 2 * p->grad_bytes + sizeof(int) * 2 * PEER_MAX;
  STAFB_CUDA_OK(cudaMalloc((void**)&p->block, bytes));
  STAFB_CUDA_OK(cudaMemset(p->block, 0, bytes));
  STAFB_CUDA_OK(cudaMalloc((void**)&p->status_d, 2 * sizeof(int)));  // status word, verdict word
  STAFB_CUDA_OK(cudaMemset(p->status_d, 0, 2 * sizeof(int)));
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

// Writes `value` into every flag word of this rank's block for `parity`, as if all peers had published step
// `value` already.  For emulating several ranks on one GPU, where their kernels run one after the other and
// must therefore never wait for each other.
extern "C" int stafb_peer_preset_flags(stafb_peer* p, void* stream, int parity, int value) {
  if (!p || parity < 0 || parity > 1) return STAFB_ERR_INVALID;
  int host[PEER_MAX];
  for (int r = 0; r < PEER_MAX; r++) host[r] = value;
  int* flags = reinterpret_cast<int*>(p->block + 2 * p->grad_bytes) + parity * PEER_MAX;
  STAFB_CUDA_OK(cudaMemcpyAsync(flags, host, sizeof(host), cudaMemcpyHostToDevice, (cudaStream_t)stream));
  STAFB_CUDA_OK(cudaStreamSynchronize((cudaStream_t)stream));
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

extern "C" int stafb_allreduce_adam(stafb_ctx* c, stafb_peer* p, void* stream, int parity, void* theta, void* mm,
                                    void* vv, double lr, double b1, double b2, double eps, int* step_d) {
  if (!c || !p || !theta || !mm || !vv || !step_d || parity < 0 || parity > 1 || !p->connected)
    return STAFB_ERR_INVALID;
  if (c->dtype != p->dtype) return STAFB_ERR_INVALID;
  PeerView pv;
  memset(&pv, 0, sizeof(pv));
  pv.rank = p->rank;
  pv.world = p->world;
  for (int r = 0; r < p->world; r++) {
    pv.grad[r] = p->peer[r] + (size_t)parity * p->grad_bytes;
    int* flags_r = reinterpret_cast<int*>(p->peer[r] + 2 * p->grad_bytes);
    pv.flag_out[r] = flags_r + parity * PEER_MAX + p->rank;
  }
  pv.flag_in = reinterpret_cast<const int*>(p->block + 2 * p->grad_bytes) + parity * PEER_MAX;
  cudaStream_t s = (cudaStream_t)stream;
  const int n = p->n, grid = (n + 255) / 256;
  if (c->dtype == STAFB_F32)
    STAFB_CUDA_OK(launch_chained(k_allreduce_adam<float>, grid, 256, 0, s, pv, n, (float*)theta, (float*)mm,
                                 (float*)vv, lr, b1, b2, (float)eps, step_d, p->wait_cycles, p->status_d));
  else
    STAFB_CUDA_OK(launch_chained(k_allreduce_adam<double>, grid, 256, 0, s, pv, n, (double*)theta, (double*)mm,
                                 (double*)vv, lr, b1, b2, eps, step_d, p->wait_cycles, p->status_d));
  return STAFB_OK;
}

// Halo exchange of a slab decomposition over NVLink peer memory.
//
// What LAMMPS' forward and reverse communication do around pair_style staf in the reference
// (lammps/USER-STAF/pair_staf.cpp:129-145,180-256: ghost atoms within one cutoff of a domain, forces on ghosts
// summed back onto their owners) for the ranks of ONE node, one rank per GPU, without a message library on the
// path of an evaluation.  The periodic box is cut into `world` slabs along one axis; rank r's neighbours are
// lo = r-1 and hi = r+1 (mod world).  Every rank keeps ONE block of device memory that its peers have mapped
// (CUDA IPC, or directly when the ranks live in one process):
//   pos_all[cap_atoms][3]   its atom array: owned atoms, then the ghosts from lo, then the ghosts from hi - the
//                           neighbours write their face atoms straight into the ghost regions;
//   frecv[2][cap_face][3]   forces on the atoms this rank sent through its lower / upper face, written by lo / hi;
//   esl[2][PEER_MAX]        per-rank energies of the current and the previous evaluation (step parity);
//   flags                   "positions from lo / hi", "forces from lo / hi", "energy of rank r": the number of the
//                           evaluation they belong to (monotonic, so nothing is ever cleared).
// An evaluation is four small launches around stafb_energy_force_domain:
//   push_positions   gather the face atoms, store them into the neighbours' arrays, publish (a few blocks; the
//                    one that finishes last publishes);
//   wait_positions   bounded wait for both neighbours (a status on a miss, never a hang);
//   return_forces    store the ghost forces into the neighbours' frecv, the energy into everybody's esl, publish;
//   collect          bounded wait, add the returned forces onto the owners, sum the energies in rank order.
// All of them read the evaluation number from a device counter that collect() advances, so the sequence can be
// captured in a CUDA graph and replayed.  Why single buffers are safe: a neighbour writes into pos_all for
// evaluation k+1 only after its own collect(k), which waited for this rank's forces of k, i.e. for the end of this
// rank's evaluation k; the energies alternate between two sets because a rank that is not a neighbour may be one
// evaluation ahead (never two: its collect(k+1) needs everybody's energy of k+1).
#include <string.h>

#include "common.cuh"

namespace stafb {

constexpr int HALO_MAX = 16;

struct HaloView {
  int rank, world, lo, hi;
  int n_own, n_from_lo, n_from_hi;  // layout of pos_all
  int n_send_lo, n_send_hi;         // atoms sent through the lower / upper face
  const int* send_lo;               // their indices among the owned atoms
  const int* send_hi;
  int dst_lo, dst_hi;               // first atom of "ghosts from hi" in lo's array / of "ghosts from lo" in hi's
  void* pos;                        // own pos_all
  void* pos_lo;                     // lo's pos_all, hi's pos_all (mapped)
  void* pos_hi;
  void* frecv;                      // own frecv[2][cap_face][3]
  void* frecv_of_lo;                // lo's frecv[1] (what lo sent through its upper face = my ghosts from lo)
  void* frecv_of_hi;                // hi's frecv[0]
  double* esl;                      // own esl[2][HALO_MAX]
  double* esl_of[HALO_MAX];         // every rank's esl (own: local pointer)
  int* flags;                       // own flags: [0] pos from lo, [1] pos from hi, [2] f from lo, [3] f from hi, [8 + r] energy of r
  int* flags_of[HALO_MAX];          // every rank's flag words
  int* step_d;                      // [1] evaluations completed
  int* status;
  int* ctr;                         // [4] arrival counters of push / return / collect, failure mark of collect
  long long wait_cycles;
  int cap_face;
};

constexpr int HALO_BLOCKS = 8;    // blocks of the kernels that move face atoms
constexpr int HALO_THREADS = 512;

// The block that arrives last at `ctr` (all others have fenced their stores before arriving) returns true and
// leaves the counter at zero for the next launch.
__device__ __forceinline__ bool h_last_block(int* ctr) {
  __shared__ int last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    last = atomicAdd(ctr, 1) == (int)gridDim.x - 1;
    if (last) { *ctr = 0; __threadfence_system(); }
  }
  __syncthreads();
  return last != 0;
}

// What the device-side choice of the ghost sets needs on top of the peers' pointers.
struct HaloPlanView {
  int rank, world, lo, hi, n_own, cap_face, cap_atoms, axis, tag;
  double L, reach;
  const void* pos;        // own atom array
  const int* types;       // species of the owned atoms
  int* send_idx;          // [2][cap_face] own lists
  int* plan;              // [8] own: n_send_lo, n_send_hi, n_from_lo, n_from_hi, dst_lo, dst_hi
  int* mail;              // own mail[2][1 + cap_face]: slot 0 written by lo, slot 1 by hi: count, species...
  int* mail_of_lo;        // lo's slot 1, hi's slot 0
  int* mail_of_hi;
  int* reply;             // own reply[2]: slot 0 written by lo, slot 1 by hi: first row of my face atoms there
  int* reply_of_lo;       // lo's reply[1], hi's reply[0]
  int* reply_of_hi;
  int* flags;             // own flag words: [4] mail from lo, [5] mail from hi, [6] reply from lo, [7] reply from hi
  int* flags_of_lo;
  int* flags_of_hi;
  int* type_all;          // [cap_atoms] species of owned + ghost atoms (caller's array)
  int* status;
  long long wait_cycles;
};

__device__ __forceinline__ int h_ld_sys(const int* p) {
  int v;
  asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void h_st_sys(int* p, int v) {
  asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// bounded wait until *p >= tag; false after `cycles`
__device__ __forceinline__ bool h_wait(const int* p, int tag, long long cycles) {
  const long long t0 = clock64();
  while (h_ld_sys(p) < tag) {
    const long long waited = clock64() - t0;
    if (waited > cycles) return false;
    if (waited > 20000) __nanosleep(100);
  }
  return true;
}

// The face atoms go to the neighbours; the block that finishes last publishes the flags.
template <class T>
__global__ void __launch_bounds__(HALO_THREADS) k_halo_push_pos(HaloView v) {
  chain_wait();
  const int tag = *reinterpret_cast<volatile int*>(v.step_d) + 1;
  const T* pos = reinterpret_cast<const T*>(v.pos);
  T* plo = reinterpret_cast<T*>(v.pos_lo);
  T* phi = reinterpret_cast<T*>(v.pos_hi);
  const int tid = blockIdx.x * blockDim.x + threadIdx.x, nth = gridDim.x * blockDim.x;
  for (int q = tid; q < 3 * v.n_send_lo; q += nth) {
    const int a = q / 3, c = q - 3 * a;
    plo[(size_t)(v.dst_lo + a) * 3 + c] = pos[(size_t)v.send_lo[a] * 3 + c];
  }
  for (int q = tid; q < 3 * v.n_send_hi; q += nth) {
    const int a = q / 3, c = q - 3 * a;
    phi[(size_t)(v.dst_hi + a) * 3 + c] = pos[(size_t)v.send_hi[a] * 3 + c];
  }
  if (h_last_block(v.ctr + 0) && threadIdx.x == 0) {
    // what leaves through my lower face arrives through lo's UPPER face
    h_st_sys(v.flags_of[v.lo] + 1, tag);
    h_st_sys(v.flags_of[v.hi] + 0, tag);
  }
}

__global__ void k_halo_wait(const int* fa, const int* fb, const int* step_d, long long cycles, int* status) {
  chain_wait();
  const int tag = *reinterpret_cast<volatile const int*>(step_d) + 1;
  if (threadIdx.x == 0) {
    const bool ok = h_wait(fa, tag, cycles) && h_wait(fb, tag, cycles);
    if (!ok) atomicCAS(status, 0, STAFB_ERR_PEER_TIMEOUT);
    __threadfence_system();
  }
}

// Ghost forces back to their owners' ranks, my energy to everybody; the block that finishes last publishes.
template <class T>
__global__ void __launch_bounds__(HALO_THREADS)
    k_halo_return(HaloView v, const T* __restrict__ force, const T* __restrict__ energy) {
  chain_wait();
  const int tag = *reinterpret_cast<volatile int*>(v.step_d) + 1;
  // my ghosts from lo are the atoms lo sent through ITS upper face: they go to lo's frecv[1]
  T* to_lo = reinterpret_cast<T*>(v.frecv_of_lo);
  T* to_hi = reinterpret_cast<T*>(v.frecv_of_hi);
  const T* g_lo = force + (size_t)v.n_own * 3;
  const T* g_hi = g_lo + (size_t)v.n_from_lo * 3;
  const int tid = blockIdx.x * blockDim.x + threadIdx.x, nth = gridDim.x * blockDim.x;
  for (int q = tid; q < 3 * v.n_from_lo; q += nth) to_lo[q] = g_lo[q];
  for (int q = tid; q < 3 * v.n_from_hi; q += nth) to_hi[q] = g_hi[q];
  if (blockIdx.x == 0 && threadIdx.x < v.world)
    v.esl_of[threadIdx.x][(tag & 1) * HALO_MAX + v.rank] = (double)energy[0];
  if (h_last_block(v.ctr + 1)) {
    if (threadIdx.x == 0) {
      h_st_sys(v.flags_of[v.lo] + 3, tag);  // lo sees "forces from hi"
      h_st_sys(v.flags_of[v.hi] + 2, tag);
    }
    if (threadIdx.x < v.world) {
      __threadfence_system();  // every publishing thread orders the block's earlier stores before its own flag
      h_st_sys(v.flags_of[threadIdx.x] + 8 + v.rank, tag);
    }
  }
}

// Every block waits for the forces of both neighbours (block 0 also for the energies of all ranks), adds its
// share of the returned forces onto the owners (an atom near both faces gets two contributions: atomics); block 0
// sums the energies in rank order.  The block that finishes last advances the evaluation number - unless a wait
// ran out somewhere, in which case the number stays as it was.
template <class T>
__global__ void __launch_bounds__(HALO_THREADS) k_halo_collect(HaloView v, T* __restrict__ force, T* __restrict__ energy_out) {
  __shared__ int ok_s;
  chain_wait();
  const int tag = *reinterpret_cast<volatile int*>(v.step_d) + 1;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  const int nwait = blockIdx.x == 0 ? v.world + 2 : 2;
  if (threadIdx.x < nwait) {
    const int* f = threadIdx.x < 2 ? v.flags + 2 + threadIdx.x : v.flags + 8 + (threadIdx.x - 2);
    if (!h_wait(f, tag, v.wait_cycles)) {
      ok_s = 0;
      atomicCAS(v.status, 0, STAFB_ERR_PEER_TIMEOUT);
      atomicExch(v.ctr + 3, 1);
    }
    __threadfence_system();
  }
  __syncthreads();
  if (ok_s) {
    const T* r_lo = reinterpret_cast<const T*>(v.frecv);
    const T* r_hi = r_lo + (size_t)v.cap_face * 3;
    const int tid = blockIdx.x * blockDim.x + threadIdx.x, nth = gridDim.x * blockDim.x;
    for (int q = tid; q < 3 * v.n_send_lo; q += nth) {
      const int a = q / 3, c = q - 3 * a;
      atomicAdd(force + (size_t)v.send_lo[a] * 3 + c, r_lo[q]);
    }
    for (int q = tid; q < 3 * v.n_send_hi; q += nth) {
      const int a = q / 3, c = q - 3 * a;
      atomicAdd(force + (size_t)v.send_hi[a] * 3 + c, r_hi[q]);
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) {
      double e = 0.0;
      for (int r = 0; r < v.world; r++) e += v.esl[(tag & 1) * HALO_MAX + r];
      energy_out[0] = (T)e;
    }
  }
  if (h_last_block(v.ctr + 2) && threadIdx.x == 0) {
    if (atomicExch(v.ctr + 3, 0) == 0) *v.step_d = tag;
  }
}

// One block.  Chooses, in index order, the owned atoms within `reach` of the lower / upper face of this rank's
// slab, keeps their indices, and stores their number and species into the neighbours' mailboxes.
template <class T>
__global__ void __launch_bounds__(1024) k_halo_select(HaloPlanView v) {
  __shared__ int wsum[2][32];
  __shared__ int base[2];
  chain_wait();
  const T* pos = reinterpret_cast<const T*>(v.pos);
  const double w = v.L / v.world;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (threadIdx.x < 2) base[threadIdx.x] = 0;
  __syncthreads();
  int* list[2] = {v.send_idx, v.send_idx + v.cap_face};
  int* mail[2] = {v.mail_of_lo, v.mail_of_hi};
  for (int i0 = 0; i0 < v.n_own; i0 += blockDim.x) {
    const int i = i0 + threadIdx.x;
    bool in[2] = {false, false};
    int sp = 0;
    if (i < v.n_own) {
      const double z = (double)pos[(size_t)i * 3 + v.axis];
      const double zw = z - floor(z / v.L) * v.L - v.rank * w;
      in[0] = zw < v.reach;
      in[1] = zw >= w - v.reach;
      sp = v.types[i];
    }
    unsigned bal[2];
    for (int f = 0; f < 2; f++) {
      bal[f] = __ballot_sync(0xffffffffu, in[f]);
      if (lane == 0) wsum[f][wid] = __popc(bal[f]);
    }
    __syncthreads();
    for (int f = 0; f < 2; f++) {
      int before = base[f];
      for (int q = 0; q < wid; q++) before += wsum[f][q];
      const int at = before + __popc(bal[f] & ((1u << lane) - 1u));
      if (in[f] && at < v.cap_face) {
        list[f][at] = i;
        mail[f][1 + at] = sp;
      }
    }
    __syncthreads();
    if (threadIdx.x < 2) {
      int tot = 0;
      for (int q = 0; q < (int)(blockDim.x >> 5); q++) tot += wsum[threadIdx.x][q];
      base[threadIdx.x] += tot;
    }
    __syncthreads();
  }
  if (threadIdx.x < 2) {
    int n = base[threadIdx.x];
    if (n > v.cap_face) { atomicCAS(v.status, 0, STAFB_ERR_CAPACITY); n = v.cap_face; }
    v.plan[threadIdx.x] = n;
    mail[threadIdx.x][0] = n;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    h_st_sys(v.flags_of_lo + 5, v.tag);  // lo reads it as "mail from hi"
    h_st_sys(v.flags_of_hi + 4, v.tag);
  }
}

// One block.  With both neighbours' mail: lays out the atom array (owned | from lo | from hi), fills the species
// of the ghosts and tells each neighbour where its face atoms start here.
__global__ void __launch_bounds__(1024) k_halo_layout(HaloPlanView v) {
  __shared__ int ok_s;
  chain_wait();
  if (threadIdx.x == 0) {
    ok_s = h_wait(v.flags + 4, v.tag, v.wait_cycles) && h_wait(v.flags + 5, v.tag, v.wait_cycles);
    if (!ok_s) atomicCAS(v.status, 0, STAFB_ERR_PEER_TIMEOUT);
    __threadfence_system();
  }
  __syncthreads();
  if (!ok_s) return;
  const int* m_lo = v.mail;
  const int* m_hi = v.mail + 1 + v.cap_face;
  int n_lo = m_lo[0], n_hi = m_hi[0];
  if (n_lo < 0 || n_hi < 0 || n_lo > v.cap_face || n_hi > v.cap_face || v.n_own + n_lo + n_hi > v.cap_atoms) {
    if (threadIdx.x == 0) atomicCAS(v.status, 0, STAFB_ERR_CAPACITY);
    n_lo = n_hi = 0;
  }
  for (int q = threadIdx.x; q < v.n_own; q += blockDim.x) v.type_all[q] = v.types[q];
  for (int q = threadIdx.x; q < n_lo; q += blockDim.x) v.type_all[v.n_own + q] = m_lo[1 + q];
  for (int q = threadIdx.x; q < n_hi; q += blockDim.x) v.type_all[v.n_own + n_lo + q] = m_hi[1 + q];
  if (threadIdx.x == 0) {
    v.plan[2] = n_lo;
    v.plan[3] = n_hi;
    // lo's upper face lands in my "from lo" rows: I am lo's hi, so it is lo's reply slot 1
    v.reply_of_lo[0] = v.n_own;
    v.reply_of_hi[0] = v.n_own + n_lo;
    __threadfence_system();
    h_st_sys(v.flags_of_lo + 7, v.tag);
    h_st_sys(v.flags_of_hi + 6, v.tag);
  }
}

// With both replies: the plan is complete on this rank.
__global__ void k_halo_plan_done(HaloPlanView v) {
  chain_wait();
  if (threadIdx.x == 0) {
    const bool ok = h_wait(v.flags + 6, v.tag, v.wait_cycles) && h_wait(v.flags + 7, v.tag, v.wait_cycles);
    if (!ok) atomicCAS(v.status, 0, STAFB_ERR_PEER_TIMEOUT);
    __threadfence_system();
    v.plan[4] = ok ? v.reply[0] : 0;
    v.plan[5] = ok ? v.reply[1] : 0;
  }
}

}  // namespace stafb

using namespace stafb;

// Block layout (device memory of this rank, mapped by the peers), offsets in bytes:
//   [ pos_all | frecv[2][cap_face][3] | esl[2][HALO_MAX] double | flags[8 + HALO_MAX] int |
//     mail[2][1 + cap_face] int | reply[2] int ]
// Every rank must use the same cap_atoms and cap_face: the peers address the block by this layout.
struct stafb_halo {
  int rank, world, dtype, cap_atoms, cap_face;
  size_t es, off_frecv, off_esl, off_flags, off_mail, off_reply, bytes;
  int* plan_d;    // [8]
  int* plan_h;    // pinned: [0..7] the plan, [8] the status word, copied behind plan_done
  cudaEvent_t plan_ev;
  int plan_no;
  int lists;      // which half of send_idx the plan in force uses (a plan under way fills the other)
  HaloPlanView pv;
  char* block;
  char* peer[HALO_MAX];
  int connected;  // 1: IPC mappings to close, 2: pointers of handles in this process
  int* send_idx;  // [2 sets][2][cap_face] device
  int* step_d;    // [1]
  int* status_d;  // [1]
  int* ctr_d;     // [4]
  void* force;    // [cap_atoms][3] local scratch for the evaluation's forces
  long long wait_cycles;
  HaloView view;
  int planned;
};

extern "C" int stafb_halo_create(stafb_ctx* c, int rank, int world, int cap_atoms, int cap_face, stafb_halo** out) {
  if (!c || !out || world < 2 || world > HALO_MAX || rank < 0 || rank >= world || cap_atoms <= 0 || cap_face <= 0)
    return STAFB_ERR_INVALID;
  stafb_halo* h = (stafb_halo*)calloc(1, sizeof(stafb_halo));
  if (!h) return STAFB_ERR_INVALID;
  h->rank = rank; h->world = world; h->dtype = c->dtype; h->cap_atoms = cap_atoms; h->cap_face = cap_face;
  h->es = c->dtype == STAFB_F32 ? 4 : 8;
  auto up = [](size_t x) { return (x + 255) / 256 * 256; };
  h->off_frecv = up(h->es * 3 * (size_t)cap_atoms);
  h->off_esl = h->off_frecv + up(h->es * 3 * 2 * (size_t)cap_face);
  h->off_flags = h->off_esl + up(sizeof(double) * 2 * HALO_MAX);
  h->off_mail = h->off_flags + up(sizeof(int) * (8 + HALO_MAX));
  h->off_reply = h->off_mail + up(sizeof(int) * 2 * (1 + (size_t)cap_face));
  h->bytes = h->off_reply + up(sizeof(int) * 2);
  STAFB_CUDA_OK(cudaMalloc((void**)&h->block, h->bytes));
  STAFB_CUDA_OK(cudaMemset(h->block, 0, h->bytes));
  STAFB_CUDA_OK(cudaMalloc((void**)&h->send_idx, sizeof(int) * 4 * (size_t)cap_face));
  STAFB_CUDA_OK(cudaMallocHost((void**)&h->plan_h, sizeof(int) * 16));
  STAFB_CUDA_OK(cudaEventCreateWithFlags(&h->plan_ev, cudaEventDisableTiming));
  STAFB_CUDA_OK(cudaMalloc((void**)&h->step_d, sizeof(int)));
  STAFB_CUDA_OK(cudaMemset(h->step_d, 0, sizeof(int)));
  STAFB_CUDA_OK(cudaMalloc((void**)&h->status_d, sizeof(int)));
  STAFB_CUDA_OK(cudaMemset(h->status_d, 0, sizeof(int)));
  STAFB_CUDA_OK(cudaMalloc((void**)&h->ctr_d, sizeof(int) * 4));
  STAFB_CUDA_OK(cudaMemset(h->ctr_d, 0, sizeof(int) * 4));
  STAFB_CUDA_OK(cudaMalloc(&h->force, h->es * 3 * (size_t)cap_atoms));
  STAFB_CUDA_OK(cudaMalloc((void**)&h->plan_d, sizeof(int) * 8));
  STAFB_CUDA_OK(cudaMemset(h->plan_d, 0, sizeof(int) * 8));
  STAFB_CUDA_OK(cudaDeviceSynchronize());
  h->peer[rank] = h->block;
  int khz = 1500000;
  cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, c->device);
  h->wait_cycles = 2LL * khz * 1000;  // about two seconds of SM clock
  if (getenv("STAFB_PEER_WAIT_MS")) h->wait_cycles = (long long)atoll(getenv("STAFB_PEER_WAIT_MS")) * khz;
  *out = h;
  return STAFB_OK;
}

extern "C" int stafb_halo_handle(stafb_halo* h, void* handle64) {
  if (!h || !handle64) return STAFB_ERR_INVALID;
  cudaIpcMemHandle_t ih;
  STAFB_CUDA_OK(cudaIpcGetMemHandle(&ih, h->block));
  memcpy(handle64, &ih, 64);
  return STAFB_OK;
}

extern "C" int stafb_halo_connect(stafb_halo* h, const void* handles) {
  if (!h || !handles) return STAFB_ERR_INVALID;
  for (int r = 0; r < h->world; r++) {
    if (r == h->rank || h->peer[r]) continue;
    cudaIpcMemHandle_t ih;
    memcpy(&ih, (const char*)handles + 64 * (size_t)r, 64);
    void* ptr = nullptr;
    STAFB_CUDA_OK(cudaIpcOpenMemHandle(&ptr, ih, cudaIpcMemLazyEnablePeerAccess));
    h->peer[r] = (char*)ptr;
  }
  h->connected = 1;
  return STAFB_OK;
}

// Ranks that live in ONE process (several emulated ranks on one GPU in a test, or one thread per GPU).
extern "C" int stafb_halo_connect_local(stafb_halo* h, stafb_halo* const* all) {
  if (!h || !all) return STAFB_ERR_INVALID;
  for (int r = 0; r < h->world; r++) {
    if (r == h->rank) continue;
    if (!all[r] || all[r]->world != h->world || all[r]->rank != r || all[r]->cap_atoms != h->cap_atoms ||
        all[r]->cap_face != h->cap_face || all[r]->dtype != h->dtype)
      return STAFB_ERR_INVALID;
    h->peer[r] = all[r]->block;
  }
  h->connected = 2;
  return STAFB_OK;
}

extern "C" void* stafb_halo_positions(stafb_halo* h) { return h ? (void*)h->block : nullptr; }
extern "C" void* stafb_halo_forces(stafb_halo* h) { return h ? h->force : nullptr; }

extern "C" int stafb_halo_set_wait_ms(stafb_halo* h, long long ms) {
  if (!h || ms < 0) return STAFB_ERR_INVALID;
  int dev = 0, khz = 1500000;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev);
  h->wait_cycles = ms * (long long)khz;
  h->view.wait_cycles = h->wait_cycles;
  return STAFB_OK;
}

static void fill_view(stafb_halo* h, int n_own, int n_from_lo, int n_from_hi, int n_send_lo, int n_send_hi,
                      int dst_off_lo, int dst_off_hi) {
  HaloView& v = h->view;
  memset(&v, 0, sizeof(v));
  v.rank = h->rank; v.world = h->world;
  v.lo = (h->rank + h->world - 1) % h->world;
  v.hi = (h->rank + 1) % h->world;
  v.n_own = n_own; v.n_from_lo = n_from_lo; v.n_from_hi = n_from_hi;
  v.n_send_lo = n_send_lo; v.n_send_hi = n_send_hi;
  v.send_lo = h->send_idx + (size_t)h->lists * 2 * h->cap_face; v.send_hi = v.send_lo + h->cap_face;
  v.dst_lo = dst_off_lo; v.dst_hi = dst_off_hi;
  v.pos = h->block;
  v.pos_lo = h->peer[v.lo]; v.pos_hi = h->peer[v.hi];
  v.frecv = h->block + h->off_frecv;
  v.frecv_of_lo = h->peer[v.lo] + h->off_frecv + h->es * 3 * (size_t)h->cap_face;  // lo's frecv[1]
  v.frecv_of_hi = h->peer[v.hi] + h->off_frecv;                                    // hi's frecv[0]
  v.esl = reinterpret_cast<double*>(h->block + h->off_esl);
  v.flags = reinterpret_cast<int*>(h->block + h->off_flags);
  for (int r = 0; r < h->world; r++) {
    v.esl_of[r] = reinterpret_cast<double*>(h->peer[r] + h->off_esl);
    v.flags_of[r] = reinterpret_cast<int*>(h->peer[r] + h->off_flags);
  }
  v.step_d = h->step_d;
  v.status = h->status_d;
  v.ctr = h->ctr_d;
  v.wait_cycles = h->wait_cycles;
  v.cap_face = h->cap_face;
  h->planned = 1;
}

// The ghost sets chosen on the device and agreed between the neighbours through their mailboxes: three launches
// (select, layout, done; ranks that share one GPU issue each of them for all ranks before the next), then _finish
// reads six integers back - the only host synchronisation of a re-plan.  No barrier between the ranks is needed:
// a neighbour stores positions by the new offsets only after this rank's layout kernel told it where, and that
// kernel runs after this rank's last evaluation under the old plan.
extern "C" int stafb_halo_plan_select(stafb_halo* h, void* stream, int n_own, const int* types_d, int axis, double L,
                                      double reach) {
  if (!h || !h->connected || n_own <= 0 || n_own > h->cap_atoms || !types_d || axis < 0 || axis > 2 || !(L > 0) ||
      !(reach > 0))
    return STAFB_ERR_INVALID;
  const double need = h->world > 2 ? reach : 2.0 * reach;
  if (L / h->world < need) return STAFB_ERR_INVALID;  // an atom would be a ghost twice on one rank
  HaloPlanView& v = h->pv;
  memset(&v, 0, sizeof(v));
  v.rank = h->rank; v.world = h->world;
  v.lo = (h->rank + h->world - 1) % h->world;
  v.hi = (h->rank + 1) % h->world;
  v.n_own = n_own; v.cap_face = h->cap_face; v.cap_atoms = h->cap_atoms; v.axis = axis;
  v.tag = ++h->plan_no;
  v.L = L; v.reach = reach;
  v.pos = h->block; v.types = types_d;
  v.send_idx = h->send_idx + (size_t)(h->lists ^ 1) * 2 * h->cap_face; v.plan = h->plan_d;
  auto mail = [&](int r, int slot) {
    return reinterpret_cast<int*>(h->peer[r] + h->off_mail) + (size_t)slot * (1 + h->cap_face);
  };
  v.mail = mail(h->rank, 0);
  v.mail_of_lo = mail(v.lo, 1);
  v.mail_of_hi = mail(v.hi, 0);
  v.reply = reinterpret_cast<int*>(h->block + h->off_reply);
  v.reply_of_lo = reinterpret_cast<int*>(h->peer[v.lo] + h->off_reply) + 1;
  v.reply_of_hi = reinterpret_cast<int*>(h->peer[v.hi] + h->off_reply);
  v.flags = reinterpret_cast<int*>(h->block + h->off_flags);
  v.flags_of_lo = reinterpret_cast<int*>(h->peer[v.lo] + h->off_flags);
  v.flags_of_hi = reinterpret_cast<int*>(h->peer[v.hi] + h->off_flags);
  v.status = h->status_d;
  v.wait_cycles = h->wait_cycles;
  cudaStream_t s = (cudaStream_t)stream;
  if (h->dtype == STAFB_F32) STAFB_CUDA_OK(launch_chained(k_halo_select<float>, 1, 1024, 0, s, v));
  else STAFB_CUDA_OK(launch_chained(k_halo_select<double>, 1, 1024, 0, s, v));
  return STAFB_OK;
}

extern "C" int stafb_halo_plan_layout(stafb_halo* h, void* stream, int* type_all_d) {
  if (!h || !h->pv.n_own || !type_all_d) return STAFB_ERR_INVALID;
  h->pv.type_all = type_all_d;
  STAFB_CUDA_OK(launch_chained(k_halo_layout, 1, 1024, 0, (cudaStream_t)stream, h->pv));
  return STAFB_OK;
}

extern "C" int stafb_halo_plan_done(stafb_halo* h, void* stream) {
  if (!h || !h->pv.n_own) return STAFB_ERR_INVALID;
  cudaStream_t s = (cudaStream_t)stream;
  STAFB_CUDA_OK(launch_chained(k_halo_plan_done, 1, 32, 0, s, h->pv));
  // the result goes to pinned memory behind an event, so that _finish need not wait for work enqueued after this
  STAFB_CUDA_OK(cudaMemcpyAsync(h->plan_h, h->plan_d, sizeof(int) * 8, cudaMemcpyDeviceToHost, s));
  STAFB_CUDA_OK(cudaMemcpyAsync(h->plan_h + 8, h->status_d, sizeof(int), cudaMemcpyDeviceToHost, s));
  STAFB_CUDA_OK(cudaEventRecord(h->plan_ev, s));
  return STAFB_OK;
}

// Waits for the three plan launches (not for anything enqueued after them) and puts the new plan in force for the
// launches that follow; counts_out[4] = n_from_lo, n_from_hi, n_send_lo, n_send_hi.  Returns the exchange's status.
// Evaluations under the old plan may be enqueued between _done and _finish: they keep the old lists and offsets.
extern "C" int stafb_halo_plan_finish(stafb_halo* h, void* stream, int* counts_out) {
  (void)stream;
  if (!h || !h->pv.n_own || !counts_out) return STAFB_ERR_INVALID;
  STAFB_CUDA_OK(cudaEventSynchronize(h->plan_ev));
  const int* p = h->plan_h;
  if (p[8]) return p[8];
  h->lists ^= 1;
  fill_view(h, h->pv.n_own, p[2], p[3], p[0], p[1], p[4], p[5]);
  counts_out[0] = p[2]; counts_out[1] = p[3]; counts_out[2] = p[0]; counts_out[3] = p[1];
  return STAFB_OK;
}

extern "C" int stafb_halo_set_plan(stafb_halo* h, void* stream, int n_own, int n_from_lo, int n_from_hi,
                                   const int* send_lo_idx_d, int n_send_lo, int dst_off_lo,
                                   const int* send_hi_idx_d, int n_send_hi, int dst_off_hi) {
  if (!h || !h->connected || n_own <= 0 || n_from_lo < 0 || n_from_hi < 0 || n_send_lo < 0 || n_send_hi < 0 ||
      dst_off_lo < 0 || dst_off_hi < 0)
    return STAFB_ERR_INVALID;
  if ((long long)n_own + n_from_lo + n_from_hi > h->cap_atoms || n_send_lo > h->cap_face || n_send_hi > h->cap_face ||
      n_from_lo > h->cap_face || n_from_hi > h->cap_face || (long long)dst_off_lo + n_send_lo > h->cap_atoms ||
      (long long)dst_off_hi + n_send_hi > h->cap_atoms)
    return STAFB_ERR_CAPACITY;
  cudaStream_t s = (cudaStream_t)stream;
  int* lists = h->send_idx + (size_t)(h->lists ^ 1) * 2 * h->cap_face;
  if (n_send_lo)
    STAFB_CUDA_OK(cudaMemcpyAsync(lists, send_lo_idx_d, sizeof(int) * n_send_lo, cudaMemcpyDeviceToDevice, s));
  if (n_send_hi)
    STAFB_CUDA_OK(cudaMemcpyAsync(lists + h->cap_face, send_hi_idx_d, sizeof(int) * n_send_hi,
                                  cudaMemcpyDeviceToDevice, s));
  h->lists ^= 1;
  fill_view(h, n_own, n_from_lo, n_from_hi, n_send_lo, n_send_hi, dst_off_lo, dst_off_hi);
  return STAFB_OK;
}

extern "C" int stafb_halo_push_positions(stafb_halo* h, void* stream) {
  if (!h || !h->planned) return STAFB_ERR_INVALID;
  cudaStream_t s = (cudaStream_t)stream;
  if (h->dtype == STAFB_F32) STAFB_CUDA_OK(launch_chained(k_halo_push_pos<float>, HALO_BLOCKS, HALO_THREADS, 0, s, h->view));
  else STAFB_CUDA_OK(launch_chained(k_halo_push_pos<double>, HALO_BLOCKS, HALO_THREADS, 0, s, h->view));
  return STAFB_OK;
}

extern "C" int stafb_halo_wait_positions(stafb_halo* h, void* stream) {
  if (!h || !h->planned) return STAFB_ERR_INVALID;
  const HaloView& v = h->view;
  STAFB_CUDA_OK(launch_chained(k_halo_wait, 1, 32, 0, (cudaStream_t)stream, (const int*)(v.flags + 0),
                               (const int*)(v.flags + 1), (const int*)v.step_d, v.wait_cycles, v.status));
  return STAFB_OK;
}

extern "C" int stafb_halo_return_forces(stafb_halo* h, void* stream, const void* force_d, const void* energy_d) {
  if (!h || !h->planned || !force_d || !energy_d) return STAFB_ERR_INVALID;
  cudaStream_t s = (cudaStream_t)stream;
  if (h->dtype == STAFB_F32)
    STAFB_CUDA_OK(launch_chained(k_halo_return<float>, HALO_BLOCKS, HALO_THREADS, 0, s, h->view, (const float*)force_d,
                                 (const float*)energy_d));
  else
    STAFB_CUDA_OK(launch_chained(k_halo_return<double>, HALO_BLOCKS, HALO_THREADS, 0, s, h->view, (const double*)force_d,
                                 (const double*)energy_d));
  return STAFB_OK;
}

extern "C" int stafb_halo_collect(stafb_halo* h, void* stream, void* force_d, void* energy_out_d) {
  if (!h || !h->planned || !force_d || !energy_out_d) return STAFB_ERR_INVALID;
  cudaStream_t s = (cudaStream_t)stream;
  if (h->dtype == STAFB_F32)
    STAFB_CUDA_OK(launch_chained(k_halo_collect<float>, HALO_BLOCKS, HALO_THREADS, 0, s, h->view, (float*)force_d, (float*)energy_out_d));
  else
    STAFB_CUDA_OK(launch_chained(k_halo_collect<double>, HALO_BLOCKS, HALO_THREADS, 0, s, h->view, (double*)force_d,
                                 (double*)energy_out_d));
  return STAFB_OK;
}

extern "C" int stafb_halo_status(stafb_halo* h) {
  if (!h) return STAFB_ERR_INVALID;
  int s = 0;
  STAFB_CUDA_OK(cudaMemcpy(&s, h->status_d, sizeof(int), cudaMemcpyDeviceToHost));
  return s;
}

extern "C" void stafb_halo_destroy(stafb_halo* h) {
  if (!h) return;
  for (int r = 0; r < h->world && h->connected == 1; r++)
    if (r != h->rank && h->peer[r]) cudaIpcCloseMemHandle(h->peer[r]);
  cudaFree(h->block); cudaFree(h->send_idx); cudaFree(h->step_d); cudaFree(h->status_d); cudaFree(h->force); cudaFree(h->plan_d); cudaFree(h->ctr_d);
  cudaFreeHost(h->plan_h);
  if (h->plan_ev) cudaEventDestroy(h->plan_ev);
  free(h);
}

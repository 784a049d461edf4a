// libstaf C API (include/staf.h) on top of the fused energy/force path.
// Mirrors the contract of the reference's libstaf/src/staf_api.cpp:39-412: type-sorted slot remap
// (staf_api.cpp:249-294), Cartesian in / Cartesian forces out in the caller's atom order, energy
// 0.5*sum(e_i), negative integer error codes, never exit().
#include <math.h>
#include <algorithm>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <string>
#include <vector>
#include "../../include/staf.h"
#include "common.cuh"

extern "C" {
int stafb_model_create(stafb_ctx* ctx, const int* shape_desc, stafb_model** out);
void stafb_model_destroy(stafb_model* m);
int stafb_model_set_counts(stafb_model* m, const int* tipos);
int stafb_energy_force_domain(stafb_ctx* ctx, stafb_model* m, void* stream, const void* positions_d,
                              const void* boxer_d, int nall, const int* type_map_d, const int* howmany_d,
                              const int* with_d, const void* theta_d, const void* emb_d, void* energy_d,
                              void* force_d, void* virial_d);
}

struct StafModel {
  std::string dir;
  StafOptions opt;
  double Rc, Rs, Ra;
  int nr, na, nt;
  std::vector<int> Fr, Fa, widths;
  std::vector<double> theta, emb;  // flat, in the layout of include/stafb.h
  // device side, (re)built when the atom count or the species counts change
  stafb_ctx* ctx;
  stafb_model* model;
  int cap_n;  // atoms (owned + ghost) the device buffers hold
  void *theta_d, *emb_d;
  // per-call staging: one pinned host block and one device block with the same layout
  //   in : pos[3*cap] | box[6] | type_map[cap] | howmany[cap] | with[cap*nr]
  //   out: force[3*cap] | energy[1] | virial[9]
  // in the computing precision and in slot order.  The caller's double arrays travel as they are (xin: x[3*nall] |
  // box[6]; fout: f[3*nall] | energy | virial[9], caller order) and two small kernels convert and permute on the
  // device, so the host only copies into and out of pinned memory.
  char *in_h, *in_d, *out_h, *out_d;
  double *xin_h, *xin_d, *fout_h, *fout_d;
  int* slot_d;  // to_slot on the device
  size_t in_bytes, out_bytes;
  cudaStream_t stream;
  std::vector<int> to_slot;
  // the species array of the previous call: while it repeats (every step of an MD run between re-neighbourings),
  // counting, validation, the slot map and its upload are skipped
  std::vector<int> type_prev, tipos_prev;
  int type_prev_null, nlocal_prev;
  // the device work of one call (copy in, kernels, copy out) captured as a CUDA graph; replayed while the call's
  // shape (atom counts per species, ghosts, list or no list) stays the same, as it does between the
  // re-neighbouring steps of an MD run
  struct GraphKey { int nall, nlocal, has_list; size_t in_used; int tipos[STAFB_MAX_TYPES]; } gkey;
  int gstate;  // 0 nothing, 1 shape seen once (ran as plain launches), 2 graph ready, -1 capture failed for this shape
  cudaGraphExec_t gexec;
};

static bool read_matrix(const std::string& path, std::vector<double>& out) {
  FILE* f = fopen(path.c_str(), "r");
  if (!f) { fprintf(stderr, "libstaf: missing %s\n", path.c_str()); return false; }
  out.clear();
  double v;
  while (fscanf(f, "%lf", &v) == 1) out.push_back(v);
  fclose(f);
  return !out.empty();
}

// STAFMLP1: magic, int32 precision, n_af, n_layers; mu[n_af]; per layer int32 act,in,out; W[in*out]; b[out]
// (libstaf/src/mlp/staf_mlp_ort.cc:99-165)
static bool read_mlp_bin(const std::string& path, int& n_af, std::vector<int>& widths, std::vector<double>& w) {
  FILE* f = fopen(path.c_str(), "rb");
  if (!f) { fprintf(stderr, "libstaf: cannot open %s\n", path.c_str()); return false; }
  char magic[8];
  int hdr[3];
  bool ok = fread(magic, 1, 8, f) == 8 && memcmp(magic, "STAFMLP1", 8) == 0 && fread(hdr, 4, 3, f) == 3;
  if (!ok) { fclose(f); fprintf(stderr, "libstaf: bad header in %s\n", path.c_str()); return false; }
  const bool dbl = hdr[0] == 1;
  n_af = hdr[1];
  const int nl = hdr[2];
  auto rd = [&](size_t n, std::vector<double>* dst) -> bool {
    if (dbl) {
      std::vector<double> t(n);
      if (fread(t.data(), 8, n, f) != n) return false;
      if (dst) dst->insert(dst->end(), t.begin(), t.end());
    } else {
      std::vector<float> t(n);
      if (fread(t.data(), 4, n, f) != n) return false;
      if (dst) dst->insert(dst->end(), t.begin(), t.end());
    }
    return true;
  };
  if (!rd(n_af, nullptr)) { fclose(f); return false; }  // mu is taken from type{k}_alpha_mu.dat
  widths.clear();
  w.clear();
  for (int l = 0; l < nl; l++) {
    int meta[3];
    if (fread(meta, 4, 3, f) != 3) { fclose(f); return false; }
    const int act = meta[0];
    if ((l < nl - 1 && act != 1) || (l == nl - 1 && act != 0)) {
      fprintf(stderr, "libstaf: %s: only tanh hidden layers and a linear output are supported\n", path.c_str());
      fclose(f);
      return false;
    }
    widths.push_back(meta[2]);
    if (!rd((size_t)meta[1] * meta[2], &w) || !rd(meta[2], &w)) { fclose(f); return false; }
  }
  fclose(f);
  return true;
}

extern "C" void staf_options_default(StafOptions* opt) {
  if (!opt) return;
  memset(opt, 0, sizeof(*opt));
  opt->mlp_backend = STAF_MLP_ORT;
  opt->device_id = 0;
  opt->precision = 0;
}

extern "C" int staf_cuda_set_device(int device_id) {
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev <= 0) return -1;
  if (device_id < 0) device_id = 0;
  device_id %= ndev;
  if (cudaSetDevice(device_id) != cudaSuccess) return -1;
  return device_id;
}

static void release_device(StafModel* m) {
  if (m->model) stafb_model_destroy(m->model);
  if (m->ctx) stafb_destroy(m->ctx);
  m->model = nullptr;
  m->ctx = nullptr;
  void* dv[] = {m->theta_d, m->emb_d, m->in_d, m->out_d, m->xin_d, m->fout_d, m->slot_d};
  for (void* q : dv) if (q) cudaFree(q);
  if (m->in_h) cudaFreeHost(m->in_h);
  if (m->out_h) cudaFreeHost(m->out_h);
  if (m->xin_h) cudaFreeHost(m->xin_h);
  if (m->fout_h) cudaFreeHost(m->fout_h);
  m->theta_d = m->emb_d = nullptr;
  m->in_d = m->out_d = m->in_h = m->out_h = nullptr;
  m->xin_h = m->xin_d = m->fout_h = m->fout_d = nullptr;
  m->slot_d = nullptr;
  m->type_prev.clear();
  m->nlocal_prev = -1;
  m->cap_n = 0;
  if (m->gexec) cudaGraphExecDestroy(m->gexec);
  m->gexec = nullptr;
  m->gstate = 0;
}

extern "C" StafModel* staf_load(const char* model_dir, const StafOptions* opt) {
  if (!model_dir) return NULL;
  StafModel* m = new StafModel();
  m->dir = model_dir;
  staf_options_default(&m->opt);
  if (opt) m->opt = *opt;
  m->ctx = nullptr; m->model = nullptr; m->cap_n = 0;
  m->theta_d = m->emb_d = nullptr;
  m->in_d = m->out_d = m->in_h = m->out_h = nullptr;
  m->xin_h = m->xin_d = m->fout_h = m->fout_d = nullptr;
  m->slot_d = nullptr;
  m->nlocal_prev = -1;
  m->type_prev_null = 0;
  m->stream = nullptr;
  m->gexec = nullptr;
  m->gstate = 0;
  memset(&m->gkey, 0, sizeof(m->gkey));
  const int dev = staf_cuda_set_device(m->opt.device_id);
  if (dev < 0) { delete m; return NULL; }
  m->opt.device_id = dev;
  // staf_jmd.cfg (keys of libstaf/vendor/jmd/nn_nn_mlp.cu:371-383), defaults of staf_api.cpp:137-147
  m->nr = 60; m->na = 1770; m->Rc = 4.5; m->Ra = 4.5; m->Rs = 2.25; m->nt = 2;
  {
    FILE* f = fopen((m->dir + "/staf_jmd.cfg").c_str(), "r");
    if (!f) f = fopen((m->dir + "/.staf_jmd_auto.cfg").c_str(), "r");
    if (f) {
      char line[512];
      while (fgets(line, sizeof(line), f)) {
        char key[256];
        double v;
        if (sscanf(line, " %255[^= ] = %lf", key, &v) == 2) {
          if (!strcmp(key, "Buffer_radial_descriptors")) m->nr = (int)v;
          else if (!strcmp(key, "Buffer_angular_descriptors")) m->na = (int)v;
          else if (!strcmp(key, "Cutoff")) m->Rc = v;
          else if (!strcmp(key, "Cutoff_Angular")) m->Ra = v;
          else if (!strcmp(key, "Hardcore_Cutoff")) m->Rs = v;
          else if (!strcmp(key, "number_of_types")) m->nt = (int)v;
        }
      }
      fclose(f);
    }
  }
  const int nt = m->nt, C = nt * (nt + 1) / 2;
  if (nt < 1 || nt > STAFB_MAX_TYPES) { delete m; return NULL; }
  std::vector<std::vector<double>> a2(nt), a3(nt), e2(nt), e3(nt), mu(nt), w(nt);
  m->Fr.resize(nt); m->Fa.resize(nt);
  for (int k = 0; k < nt; k++) {
    char p[64];
    auto path = [&](const char* suffix) { snprintf(p, sizeof(p), "/type%d_%s", k, suffix); return m->dir + p; };
    int n_af = 0;
    std::vector<int> widths;
    snprintf(p, sizeof(p), "/mlp_type%d.bin", k);
    const std::string bin_path = m->dir + p;
    if (!read_matrix(path("alpha_2body.dat"), a2[k]) || !read_matrix(path("alpha_3body.dat"), a3[k]) ||
        !read_matrix(path("type_emb_2b_sq.dat"), e2[k]) || !read_matrix(path("type_emb_3b_sq.dat"), e3[k]) ||
        !read_matrix(path("alpha_mu.dat"), mu[k]) || !read_mlp_bin(bin_path, n_af, widths, w[k])) {
      delete m;
      return NULL;
    }
    m->Fr[k] = (int)a2[k].size() / nt;
    m->Fa[k] = (int)a3[k].size() / (3 * C);
    if (k == 0) m->widths = widths;
    if (widths != m->widths || n_af != m->Fr[k] + m->Fa[k] || (int)mu[k].size() != n_af ||
        (int)e2[k].size() != nt * m->Fr[k] || (int)e3[k].size() != C * m->Fa[k] ||
        (int)widths.size() > STAFB_MAX_DENSE || widths.back() != 1) {
      fprintf(stderr, "libstaf: inconsistent model files for type %d in %s\n", k, model_dir);
      delete m;
      return NULL;
    }
  }
  for (int k = 0; k < nt; k++) {
    m->theta.insert(m->theta.end(), a2[k].begin(), a2[k].end());
    m->theta.insert(m->theta.end(), a3[k].begin(), a3[k].end());
    m->theta.insert(m->theta.end(), mu[k].begin(), mu[k].end());
    m->theta.insert(m->theta.end(), w[k].begin(), w[k].end());
    m->emb.insert(m->emb.end(), e2[k].begin(), e2[k].end());
    m->emb.insert(m->emb.end(), e3[k].begin(), e3[k].end());
  }
  return m;
}


template <class T>
static void upload(void* dst, const std::vector<double>& src) {
  std::vector<T> t(src.begin(), src.end());
  cudaMemcpy(dst, t.data(), sizeof(T) * t.size(), cudaMemcpyHostToDevice);
}

static size_t al16(size_t x) { return (x + 15) & ~(size_t)15; }

// Offsets inside the staging blocks for a capacity of `cap` atoms.
struct StageLayout {
  size_t pos, box, tmap, how, with, in_total, force, energy, virial, out_total;
};
static StageLayout stage_layout(size_t es, size_t cap, size_t nr) {
  StageLayout L;
  size_t o = 0;
  L.pos = o; o = al16(o + es * 3 * cap);
  L.box = o; o = al16(o + es * 6);
  L.tmap = o; o = al16(o + 4 * cap);
  L.how = o; o = al16(o + 4 * cap);
  L.with = o; o = al16(o + 4 * cap * nr);
  L.in_total = o;
  o = 0;
  L.force = o; o = al16(o + es * 3 * cap);
  L.energy = o; o = al16(o + es);
  L.virial = o; o = al16(o + es * 9);
  L.out_total = o;
  return L;
}

// (Re)creates the device side when more atoms arrive than the buffers hold; the species counts of the
// owned atoms are set per call with stafb_model_set_counts, which allocates nothing.
static int ensure_device(StafModel* m, int nall, const std::vector<int>& tipos) {
  const size_t es = m->opt.precision == 1 ? 8 : 4;
  if (!m->ctx || nall > m->cap_n) {
    release_device(m);
    const int cap = nall + nall / 4 + 64;  // head-room: owned and ghost counts drift from step to step in MD
    if (stafb_create(&m->ctx, m->opt.precision == 1 ? STAFB_F64 : STAFB_F32, m->Rc, m->Rs, m->Ra, m->nr, m->na, cap,
                     1) != STAFB_OK)
      return -1;
    m->cap_n = cap;
    const StageLayout L = stage_layout(es, (size_t)cap, (size_t)m->nr);
    m->in_bytes = L.in_total;
    m->out_bytes = L.out_total;
    if (cudaMalloc(&m->theta_d, es * m->theta.size()) != cudaSuccess ||
        cudaMalloc(&m->emb_d, es * m->emb.size()) != cudaSuccess ||
        cudaMalloc((void**)&m->in_d, L.in_total) != cudaSuccess ||
        cudaMalloc((void**)&m->out_d, L.out_total) != cudaSuccess ||
        cudaMallocHost((void**)&m->in_h, L.in_total) != cudaSuccess ||
        cudaMallocHost((void**)&m->out_h, L.out_total) != cudaSuccess ||
        cudaMalloc((void**)&m->xin_d, sizeof(double) * (3 * (size_t)cap + 8)) != cudaSuccess ||
        cudaMalloc((void**)&m->fout_d, sizeof(double) * (3 * (size_t)cap + 16)) != cudaSuccess ||
        cudaMalloc((void**)&m->slot_d, sizeof(int) * (size_t)cap) != cudaSuccess ||
        cudaMallocHost((void**)&m->xin_h, sizeof(double) * (3 * (size_t)cap + 8)) != cudaSuccess ||
        cudaMallocHost((void**)&m->fout_h, sizeof(double) * (3 * (size_t)cap + 16)) != cudaSuccess)
      return -1;
    if (!m->stream && cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking) != cudaSuccess) return -1;
    if (es == 8) { upload<double>(m->theta_d, m->theta); upload<double>(m->emb_d, m->emb); }
    else { upload<float>(m->theta_d, m->theta); upload<float>(m->emb_d, m->emb); }
    int sd[20] = {0};
    sd[0] = m->nt;
    for (int t = 0; t < m->nt; t++) { sd[1 + t] = tipos[t]; sd[5 + t] = m->Fr[t]; sd[9 + t] = m->Fa[t]; }
    sd[13] = (int)m->widths.size();
    for (size_t l = 0; l < m->widths.size(); l++) sd[14 + l] = m->widths[l];
    if (stafb_model_create(m->ctx, sd, &m->model) != STAFB_OK) return -1;
  }
  return stafb_model_set_counts(m->model, tipos.data()) == STAFB_OK ? 0 : -1;
}

// Caller order, double -> slot order, computing precision (positions and box), and back (forces, energy, virial).
template <class T>
__global__ void k_stage_in(int nall, const double* __restrict__ xin, const int* __restrict__ slot, T* __restrict__ pos,
                           T* __restrict__ box) {
  const int q = blockIdx.x * blockDim.x + threadIdx.x;
  if (q < 3 * nall) {
    const int i = q / 3, c = q - 3 * i;
    pos[3 * (size_t)slot[i] + c] = (T)xin[q];
  }
  if (q < 6) box[q] = (T)xin[3 * (size_t)nall + q];
}
template <class T>
__global__ void k_stage_out(int nall, const T* __restrict__ force, const T* __restrict__ energy,
                            const T* __restrict__ virial, const int* __restrict__ slot, double* __restrict__ fout) {
  const int q = blockIdx.x * blockDim.x + threadIdx.x;
  if (q < 3 * nall) {
    const int i = q / 3, c = q - 3 * i;
    fout[q] = (double)force[3 * (size_t)slot[i] + c];
  }
  if (q == 0) fout[3 * (size_t)nall] = (double)energy[0];
  if (q < 9) fout[3 * (size_t)nall + 1 + q] = (double)virial[q];
}

// Shared body of staf_compute and staf_compute_domain.  Slots: owned atoms type-sorted in
// [0, nlocal), ghosts appended in the caller's order (libstaf/src/staf_api.cpp:249-294).
template <class T>
static int compute_impl(StafModel* m, int nlocal, int nghost, const double* x, const double* box, const int* type,
                        const int* howmany, const int* with, int maxneigh, bool use_ghosts, double* e_rank,
                        double* f, double* virial) {
  const int nt = m->nt, nr = m->nr;
  const int nall = use_ghosts ? nlocal + (nghost > 0 ? nghost : 0) : nlocal;
  const bool same_types = m->ctx && m->nlocal_prev == nlocal && (int)m->to_slot.size() == nall &&
                          m->type_prev_null == (type == nullptr) &&
                          (!type || memcmp(type, m->type_prev.data(), sizeof(int) * (size_t)nall) == 0);
  std::vector<int> tipos(nt, 0);
  if (same_types) {
    tipos = m->tipos_prev;
  } else {
    for (int i = 0; i < nall; i++) {
      const int sp = type ? type[i] : 0;
      if (sp < 0 || sp >= nt) { fprintf(stderr, "staf_compute: unsupported type %d at atom %d\n", sp, i); return -8; }
      if (i < nlocal) tipos[sp]++;
    }
  }
  const int cap_before = m->cap_n;
  if (ensure_device(m, nall, tipos) != 0) return -1;
  const bool remap = !same_types || m->cap_n != cap_before;  // new buffers are empty
  const StageLayout L = stage_layout(sizeof(T), (size_t)m->cap_n, (size_t)nr);
  int* tmap_h = reinterpret_cast<int*>(m->in_h + L.tmap);
  int* how_h = reinterpret_cast<int*>(m->in_h + L.how);
  int* with_h = reinterpret_cast<int*>(m->in_h + L.with);
  cudaStream_t s = m->stream;
  if (remap) {
    std::vector<int> cursor(nt, 0);
    for (int t = 1; t < nt; t++) cursor[t] = cursor[t - 1] + tipos[t - 1];
    m->to_slot.resize(nall);
    for (int i = 0; i < nall; i++) {
      const int sp = type ? type[i] : 0;
      const int slot = i < nlocal ? cursor[sp]++ : i;
      m->to_slot[i] = slot;
      tmap_h[slot] = sp;
    }
    // to_slot itself is pageable: stage it behind the type map in the pinned block (the list area is rewritten
    // after this copy has been enqueued only when a list is given, and then it is ordered behind it on the stream)
    if (cudaMemcpyAsync(m->in_d + L.tmap, tmap_h, sizeof(int) * (size_t)nall, cudaMemcpyHostToDevice, s) !=
            cudaSuccess ||
        cudaMemcpyAsync(m->slot_d, m->to_slot.data(), sizeof(int) * (size_t)nall, cudaMemcpyHostToDevice, s) !=
            cudaSuccess ||
        cudaStreamSynchronize(s) != cudaSuccess)
      return -14;
    m->type_prev_null = type == nullptr;
    if (type) m->type_prev.assign(type, type + nall);
    else m->type_prev.clear();
    m->tipos_prev = tipos;
    m->nlocal_prev = nlocal;
  }
  memcpy(m->xin_h, x, sizeof(double) * 3 * (size_t)nall);
  for (int a = 0; a < 6; a++) m->xin_h[3 * (size_t)nall + a] = box[a];
  size_t list_bytes = 0;
  if (howmany) {
    // caller's rows -> slot order and slot indices (staf_api.cpp:304-347)
    for (int i = 0; i < nlocal; i++) {
      const int slot = m->to_slot[i];
      int nn = howmany[i];
      if (nn < 0) nn = 0;
      if (nn > nr) nn = nr;
      if (nn > maxneigh) nn = maxneigh;
      how_h[slot] = nn;
      int* row = with_h + (size_t)slot * nr;
      for (int k = 0; k < nn; k++) {
        const int j = with[(size_t)i * maxneigh + k];
        if (j < 0 || j >= nall) {
          fprintf(stderr, "staf_compute: neighbor index %d out of range [0,%d)\n", j, nall);
          return -9;
        }
        row[k] = m->to_slot[j];
      }
    }
    list_bytes = L.with + 4 * (size_t)nlocal * nr - L.how;
  }
  const int nb = (3 * nall + 255) / 256;
  auto enqueue = [&]() -> int {
    if (cudaMemcpyAsync(m->xin_d, m->xin_h, sizeof(double) * (3 * (size_t)nall + 6), cudaMemcpyHostToDevice, s) !=
        cudaSuccess)
      return -14;
    if (list_bytes &&
        cudaMemcpyAsync(m->in_d + L.how, m->in_h + L.how, list_bytes, cudaMemcpyHostToDevice, s) != cudaSuccess)
      return -14;
    k_stage_in<T><<<nb, 256, 0, s>>>(nall, m->xin_d, m->slot_d, reinterpret_cast<T*>(m->in_d + L.pos),
                                     reinterpret_cast<T*>(m->in_d + L.box));
    const int rc = stafb_energy_force_domain(
        m->ctx, m->model, s, m->in_d + L.pos, m->in_d + L.box, nall, reinterpret_cast<const int*>(m->in_d + L.tmap),
        howmany ? reinterpret_cast<const int*>(m->in_d + L.how) : nullptr,
        howmany ? reinterpret_cast<const int*>(m->in_d + L.with) : nullptr, m->theta_d, m->emb_d, m->out_d + L.energy,
        m->out_d + L.force, m->out_d + L.virial);
    if (rc != STAFB_OK) return rc == STAFB_ERR_CUDA ? -14 : -13;
    k_stage_out<T><<<nb, 256, 0, s>>>(nall, reinterpret_cast<const T*>(m->out_d + L.force),
                                      reinterpret_cast<const T*>(m->out_d + L.energy),
                                      reinterpret_cast<const T*>(m->out_d + L.virial), m->slot_d, m->fout_d);
    if (cudaMemcpyAsync(m->fout_h, m->fout_d, sizeof(double) * (3 * (size_t)nall + 10), cudaMemcpyDeviceToHost, s) !=
        cudaSuccess)
      return -14;
    return 0;
  };
  StafModel::GraphKey key;
  memset(&key, 0, sizeof(key));
  key.nall = nall; key.nlocal = nlocal; key.has_list = howmany != nullptr; key.in_used = list_bytes;
  for (int t = 0; t < nt; t++) key.tipos[t] = tipos[t];
  if (m->gstate == 0 || memcmp(&key, &m->gkey, sizeof(key)) != 0) {
    if (m->gexec) { cudaGraphExecDestroy(m->gexec); m->gexec = nullptr; }
    m->gkey = key;
    m->gstate = 0;
  }
  static const bool no_graph = getenv("STAFB_NO_STEP_GRAPH") != nullptr;
  if (m->gstate == 2) {
    if (cudaGraphLaunch(m->gexec, s) != cudaSuccess) return -14;
  } else if (m->gstate == 1 && !no_graph) {
    cudaGraph_t g = nullptr;
    int rc = 0;
    bool ok = cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
    if (ok) {
      rc = enqueue();
      ok = cudaStreamEndCapture(s, &g) == cudaSuccess && rc == 0 && g != nullptr;
    }
    if (ok) ok = cudaGraphInstantiate(&m->gexec, g, 0) == cudaSuccess;
    if (g) cudaGraphDestroy(g);
    if (ok) {
      m->gstate = 2;
      if (cudaGraphLaunch(m->gexec, s) != cudaSuccess) return -14;
    } else {
      cudaGetLastError();
      m->gexec = nullptr;
      m->gstate = -1;
      rc = enqueue();
      if (rc != 0) return rc;
    }
  } else {
    const int rc = enqueue();
    if (rc != 0) return rc;
    if (m->gstate == 0) m->gstate = 1;
  }
  const int st = stafb_status(m->ctx, s);  // synchronises the stream
  if (st == STAFB_ERR_RADIAL_OVERFLOW) return -11;
  if (st == STAFB_ERR_ANGULAR_OVERFLOW) return -12;
  if (st == STAFB_ERR_BAD_BOX) return -7;
  if (st == STAFB_ERR_CUDA) return -14;
  if (st != STAFB_OK && st != STAFB_ERR_NONFINITE) return -13;
  const double* o = m->fout_h + 3 * (size_t)nall;
  const double energy = o[0];
  if (!isfinite(energy))  // as staf_api.cpp:378-381
    fprintf(stderr, "staf_compute: non-finite energy=%g nlocal=%d nghost=%d\n", energy, nlocal, nghost);
  if (e_rank) *e_rank = energy;
  if (f) memcpy(f, m->fout_h, sizeof(double) * 3 * (size_t)nall);
  if (virial) {
    // diagonal only, like the reference (staf_api.cpp:398-403)
    virial[0] = o[1]; virial[1] = o[5]; virial[2] = o[9];
    virial[3] = virial[4] = virial[5] = 0.0;
  }
  return 0;
}

static int compute_checked(StafModel* m, int nlocal, int nghost, const double* x, const double* box, const int* type,
                           const int* howmany, const int* with, int maxneigh, bool use_ghosts, double* e_rank,
                           double* f, double* virial) {
  if (!m || !x || !box) return -1;
  if (nlocal <= 0) return -3;
  if (howmany && (!with || maxneigh <= 0)) return -1;
  if (box[0] == 0.0 || box[3] == 0.0 || box[5] == 0.0) return -7;
  if (cudaSetDevice(m->opt.device_id) != cudaSuccess) return -14;
  if (m->opt.precision == 1)
    return compute_impl<double>(m, nlocal, nghost, x, box, type, howmany, with, maxneigh, use_ghosts, e_rank, f,
                                virial);
  return compute_impl<float>(m, nlocal, nghost, x, box, type, howmany, with, maxneigh, use_ghosts, e_rank, f, virial);
}

extern "C" int staf_compute(StafModel* m, int nlocal, int nghost, const double* x, const double* box,
                            const int* type, const int* howmany, const int* with, int maxneigh, double* e_rank,
                            double* f, double* virial) {
  // howmany == NULL: own minimum-image list over the nlocal atoms, nghost ignored (staf_api.cpp:211-212)
  return compute_checked(m, nlocal, nghost, x, box, type, howmany, with, maxneigh, howmany != NULL, e_rank, f,
                         virial);
}

extern "C" int staf_compute_domain(StafModel* m, int nlocal, int nghost, const double* x, const double* box,
                                   const int* type, double* e_rank, double* f, double* virial) {
  return compute_checked(m, nlocal, nghost, x, box, type, NULL, NULL, 0, true, e_rank, f, virial);
}

extern "C" void staf_free(StafModel* m) {
  if (!m) return;
  cudaSetDevice(m->opt.device_id);
  release_device(m);
  if (m->stream) cudaStreamDestroy(m->stream);
  delete m;
}

// ---------------------------------------------------------------------------- pluggable-MLP API (staf_mlp.h)
#include "../../include/staf_mlp.h"

extern "C" int stafb_mlp_eval(stafb_ctx* ctx, stafb_model* m, void* stream, const void* af_d, const void* theta_d,
                              const void* emb_d, void* energy_d, void* dE_daf_d);
extern "C" int stafb_status(stafb_ctx* ctx, void* stream);

// The reference's StafMlp (libstaf/src/mlp/staf_mlp_ort.cc:24-60) owns an ONNX session or the Dense weights of
// every type; here it is the loaded model plus two device arrays [atoms][Fmax] for the fingerprints and dE/dAF.
struct StafMlp {
  StafModel* m;
  void *af_d, *nd_d, *e_d;
  size_t cap_rows;
  std::vector<char> host;  // packing scratch, rows of Fmax
};

extern "C" StafMlp* staf_mlp_create(StafMlpBackend backend, const char* model_dir, int precision, int device_id) {
  if (precision != 0 && precision != 1) return NULL;
  StafOptions opt;
  staf_options_default(&opt);
  opt.mlp_backend = backend;
  opt.precision = precision;
  opt.device_id = device_id;
  StafModel* m = staf_load(model_dir, &opt);
  if (!m) return NULL;
  StafMlp* p = new StafMlp();
  p->m = m;
  p->af_d = p->nd_d = p->e_d = nullptr;
  p->cap_rows = 0;
  return p;
}

template <class T>
static int mlp_eval_impl(StafMlp* p, StafMlpEval* io, const T* af, T* energy, T* dE) {
  StafModel* m = p->m;
  if (!af || !energy || !dE || !io->n_atoms || !io->n_af || io->n_type != m->nt) return io->n_type != m->nt ? -2 : -1;
  std::vector<int> tipos(m->nt);
  int N = 0, Fmax = 0;
  for (int t = 0; t < m->nt; t++) {
    if (io->n_af[t] != m->Fr[t] + m->Fa[t] || io->n_atoms[t] < 0) return -2;
    tipos[t] = io->n_atoms[t];
    N += tipos[t];
    Fmax = std::max(Fmax, m->Fr[t] + m->Fa[t]);
  }
  if (N <= 0) return -1;
  if (cudaSetDevice(m->opt.device_id) != cudaSuccess) return -14;
  if (ensure_device(m, N, tipos) != 0) return -1;
  const size_t rows = (size_t)N;
  if (rows > p->cap_rows) {
    cudaFree(p->af_d); cudaFree(p->nd_d); cudaFree(p->e_d);
    p->af_d = p->nd_d = p->e_d = nullptr;
    p->cap_rows = 0;
    const size_t cap = rows + rows / 4 + 64;
    if (cudaMalloc(&p->af_d, sizeof(T) * cap * Fmax) != cudaSuccess ||
        cudaMalloc(&p->nd_d, sizeof(T) * cap * Fmax) != cudaSuccess || cudaMalloc(&p->e_d, sizeof(T)) != cudaSuccess)
      return -1;
    p->cap_rows = cap;
  }
  // packed [n_atoms_k][n_af_k] per type -> rows of Fmax in type order (the model's atom order)
  p->host.resize(sizeof(T) * rows * Fmax);
  T* h = reinterpret_cast<T*>(p->host.data());
  {
    size_t src = 0, row = 0;
    for (int t = 0; t < m->nt; t++)
      for (int a = 0; a < tipos[t]; a++, row++) {
        const int F = io->n_af[t];
        for (int i = 0; i < Fmax; i++) h[row * Fmax + i] = i < F ? af[src + i] : T(1);
        src += F;
      }
  }
  if (cudaMemcpyAsync(p->af_d, h, sizeof(T) * rows * Fmax, cudaMemcpyHostToDevice, m->stream) != cudaSuccess) return -14;
  const int rc = stafb_mlp_eval(m->ctx, m->model, m->stream, p->af_d, m->theta_d, m->emb_d, p->e_d, p->nd_d);
  if (rc != STAFB_OK) return rc == STAFB_ERR_CUDA ? -14 : -1;
  T e = T(0);
  if (cudaMemcpyAsync(h, p->nd_d, sizeof(T) * rows * Fmax, cudaMemcpyDeviceToHost, m->stream) != cudaSuccess ||
      cudaMemcpyAsync(&e, p->e_d, sizeof(T), cudaMemcpyDeviceToHost, m->stream) != cudaSuccess)
    return -14;
  const int st = stafb_status(m->ctx, m->stream);  // waits for the stream
  if (st == STAFB_ERR_CUDA) return -14;
  if (st != STAFB_OK) return -13;
  {
    size_t dst = 0, row = 0;
    for (int t = 0; t < m->nt; t++)
      for (int a = 0; a < tipos[t]; a++, row++) {
        const int F = io->n_af[t];
        for (int i = 0; i < F; i++) dE[dst + i] = h[row * Fmax + i];
        dst += F;
      }
  }
  energy[0] = e;
  return 0;
}

extern "C" int staf_mlp_eval(StafMlp* mlp, StafMlpEval* io) {
  if (!mlp || !mlp->m || !io) return -1;
  if (mlp->m->opt.precision == 1) return mlp_eval_impl<double>(mlp, io, io->af_f64, io->energy_f64, io->dE_daf_f64);
  return mlp_eval_impl<float>(mlp, io, io->af_f32, io->energy_f32, io->dE_daf_f32);
}

extern "C" void staf_mlp_destroy(StafMlp* mlp) {
  if (!mlp) return;
  if (mlp->m) cudaSetDevice(mlp->m->opt.device_id);
  cudaFree(mlp->af_d); cudaFree(mlp->nd_d); cudaFree(mlp->e_d);
  staf_free(mlp->m);
  delete mlp;
}

extern "C" int staf_mlp_ntypes(const StafMlp* mlp) { return mlp && mlp->m ? mlp->m->nt : 0; }
extern "C" int staf_mlp_n_af(const StafMlp* mlp, int type) {
  if (!mlp || !mlp->m || type < 0 || type >= mlp->m->nt) return 0;
  return mlp->m->Fr[type] + mlp->m->Fa[type];
}
extern "C" int staf_mlp_precision(const StafMlp* mlp) { return mlp && mlp->m ? mlp->m->opt.precision : 0; }

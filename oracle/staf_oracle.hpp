// CPU oracle for the STAF descriptor / fingerprint / force / gradient hot path.
//
// TEST INFRASTRUCTURE ONLY.  This header restates, on the CPU, the arithmetic of the
// reference's CUDA custom ops (paths relative to the reference project root):
//   neighbour list      STAF/src/descriptor_builder/celle_gpu.cu.cc:40-260,
//                       STAF/src/descriptor_builder/reforce.cc:283-340
//   descriptors         STAF/src/descriptor_builder/reforce.cu.cc:17-236,
//                       STAF/src/descriptor_builder/reforce.cc:101-125
//   fingerprints (AF)   STAF/src/fingerprint/{rad,ang}/reforce.cu.cc
//   forces              STAF/src/force/{rad,ang}/reforce.cu.cc:45-136 / 48-232
//   d/d(alpha) of AF    STAF/src/grad_finger/{rad,ang}/reforce.cu.cc
//   backward of forces  STAF/src/grad_force/{rad,ang}/reforce.cu.cc:46-123 / 47-231
//   MLP head and loss   STAF/staf_models/staf_model.py:168-258,
//                       libstaf/src/mlp/staf_mlp_ort.cc:196-242
// It is the checker the GPU library is compared against and the timed CPU baseline.
// The shipped library never includes, links or calls anything in this directory.
//
// Pinning: the MLP forward/gradient is checked against the reference's own
// eval_type_native, the neighbour list against the reference's CPU cell list
// (both compiled from the reference tree into oracle/_ref), the energy of the
// reference's frame pos_0 with its exported model against the recorded value
// -102.2588, and every gradient against finite differences in double precision.
//
// Conventions: per-term arithmetic is done in T (float or double) exactly in the
// reference's expression order; sums over neighbours / triplets / atoms are
// accumulated in double so that the oracle is a well-conditioned target for a
// GPU result that sums in a different order.
#pragma once
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>
#include <algorithm>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace stafo {

enum { MAX_TYPES = 4, MAX_DENSE = 6 };
enum Status { OK = 0, ERR_RADIAL_OVERFLOW = 1, ERR_ANGULAR_OVERFLOW = 2, ERR_CELL_OVERFLOW = 3, ERR_BAD_BOX = 4 };

// Per-thread double accumulators merged in thread order (deterministic for a
// fixed thread count).
struct ThreadAcc {
  std::vector<std::vector<double>> bufs;
  size_t n;
  explicit ThreadAcc(size_t n_) : n(n_) {
    int nth = 1;
#ifdef _OPENMP
    nth = omp_get_max_threads();
#endif
    bufs.assign(nth, std::vector<double>(n, 0.0));
  }
  double* mine() {
    int t = 0;
#ifdef _OPENMP
    t = omp_get_thread_num();
#endif
    return bufs[t].data();
  }
  void merge_into(double* dst) {
    for (auto& b : bufs)
      for (size_t i = 0; i < n; i++) dst[i] += b[i];
  }
};

inline void atomic_add(double* p, double v) {
#pragma omp atomic
  *p += v;
}

template <class T> inline T PIc() { return T(3.141592654); }  // reforce.cu.cc:15 (literal, not pi)

template <class T>
struct DescCfg {
  T Rc, Rs, Ra;
  int nr, na;
  T coeffA, coeffB, coeffC, pow_alpha, pow_beta;
};

// Repulsive-core coefficients: descriptor_builder/reforce.cc:101-125.
template <class T>
void fill_repulsion(DescCfg<T>& c) {
  const T PI = PIc<T>();
  T alpha = 1., beta = -30.;
  c.pow_alpha = alpha;
  c.pow_beta = beta;
  T rs = c.Rs, rc = c.Rc;
  T f = 0.5 * (std::cos(PI * rs / rc) + 1);
  T f1 = -0.5 * PI / rc * std::sin(PI * rs / rc);
  T f2_red = -0.5 * ((PI / rc) * (PI / rc)) * std::cos(PI * rs / rc) * (rs * rs);
  T gamma_red = 1. / (alpha - beta) * alpha - 1;
  T delta_red = 1. / (alpha - beta) * (f * (alpha - beta) - f1 * rs - f * alpha);
  T eta_red = -alpha / (alpha - beta);
  T epsilon_red = 1. / (alpha - beta) * (rs * f1 + alpha * f);
  T c2_red = alpha * (alpha + 1) * delta_red + beta * (beta + 1) * epsilon_red;
  T c1_red = alpha * (alpha + 1) * gamma_red + beta * (beta + 1) * eta_red;
  c.coeffC = (f2_red - c2_red) / c1_red;
  T eta = -alpha * std::pow(rs, beta) / (alpha - beta);
  T epsilon = std::pow(rs, beta) / (alpha - beta) * (rs * f1 + alpha * f);
  c.coeffB = eta * c.coeffC + epsilon;
  T gamma = std::pow(rs, alpha) / (alpha - beta) * alpha - std::pow(rs, alpha);
  T delta = std::pow(rs, alpha) / (alpha - beta) * (f * (alpha - beta) - f1 * rs - f * alpha);
  c.coeffA = gamma * c.coeffC + delta;
}

// Upper-triangular inverse box: descriptor_builder/reforce.cc:283-299.
template <class T>
void inverse_box(const T* B, T* I) {
  I[0] = T(1.) / B[0];
  I[1] = -B[1] / (B[0] * B[3]);
  I[2] = (B[1] * B[4]) / (B[0] * B[3] * B[5]) - B[2] / (B[0] * B[5]);
  I[3] = T(1.) / B[3];
  I[4] = -B[4] / (B[3] * B[5]);
  I[5] = T(1.) / B[5];
}

// Cell counts per axis: celle_gpu.cu.cc:208-228.
template <class T>
void cell_counts(const T* box, T cutoff, int N, int* nx, int* ny, int* nz) {
  T volume = box[0] * box[3] * box[5];
  int cx = (int)(volume / (std::sqrt(box[3] * box[3] * box[5] * box[5] + box[5] * box[5] * box[1] * box[1] +
                                     box[3] * box[3] * box[2] * box[2] + box[4] * box[4] * box[1] * box[1]) *
                           cutoff));
  int cy = (int)(volume / (box[0] * std::sqrt(box[5] * box[5] + box[4] * box[4]) * cutoff));
  int cz = (int)(volume / (box[0] * box[3] * cutoff));
  while ((cx * cy * cz > 27) && (cx * cy * cz > N)) {
    int* m = (cx > cy ? &cx : &cy);
    m = (*m > cz ? m : &cz);
    (*m)--;
  }
  if (cx < 3) cx = 3;
  if (cy < 3) cy = 3;
  if (cz < 3) cz = 3;
  *nx = cx; *ny = cy; *nz = cz;
}

// MIC displacement r_a - r_b in Cartesian space from fractional coordinates
// (rint in fractional space, then H*ds): celle_gpu.cu.cc:96-109, reforce.cu.cc:56-69.
template <class T>
inline void mic(const T* box, const T* sa, const T* sb, T* d) {
  T ox = sa[0] - sb[0], oy = sa[1] - sb[1], oz = sa[2] - sb[2];
  ox -= std::rint(ox);
  oy -= std::rint(oy);
  oz -= std::rint(oz);
  d[0] = box[0] * ox + box[1] * oy + box[2] * oz;
  d[1] = box[3] * oy + box[4] * oz;
  d[2] = box[5] * oz;
}

// Neighbour list of one frame.  Discovery order = neighbour-cell loop (x outer,
// y, z inner, offsets -1,0,1: celle_gpu.cu.cc:61-82) then slot order inside the
// cell; the reference's slot order is atomicAdd arrival (celle_gpu.cu.cc:197-200),
// restated here as ascending atom index.  Stable insertion sort by dist2 with a
// strict '>' (celle_gpu.cu.cc:128-152).  Returns OK or an overflow status; the
// reference exits the process on radial overflow (reforce.cc:324-340) and
// silently drops atoms beyond MAX_PARTICLE_CELLS (celle_gpu.cu.cc:197-200).
template <class T>
int neighbour_list(T Rc, int nr, int N, const T* pos, const T* box, T* frac, int* with, int* howmany, T* with_d2,
                   int* ncell_out /*3 or null*/) {
  if (!(box[0] != 0 && box[3] != 0 && box[5] != 0)) return ERR_BAD_BOX;
  T I[6];
  inverse_box(box, I);
  for (int p = 0; p < N; p++) {  // celle_gpu.cu.cc:11-28
    T px = pos[3 * p], py = pos[3 * p + 1], pz = pos[3 * p + 2];
    frac[3 * p + 0] = (I[0] * px + I[1] * py + I[2] * pz);
    frac[3 * p + 1] = (I[3] * py + I[4] * pz);
    frac[3 * p + 2] = (I[5] * pz);
  }
  int nx, ny, nz;
  cell_counts(box, Rc, N, &nx, &ny, &nz);
  if (ncell_out) { ncell_out[0] = nx; ncell_out[1] = ny; ncell_out[2] = nz; }
  int MPC = N / 3;  // reforce.cc:306-309
  if (MPC < 1) MPC = 1;
  if (MPC > 256) MPC = 256;
  T sx = T(1.) / (T)nx, sy = T(1.) / (T)ny, sz = T(1.) / (T)nz;
  int ncell = nx * ny * nz;
  std::vector<std::vector<int>> cells(ncell);
  int status = OK;
  for (int t = 0; t < N; t++) {  // celle_gpu.cu.cc:176-201
    int px = (int)std::floor(frac[3 * t] / sx);
    px = px % nx;
    while (px < 0) px += nx;
    int py = (int)std::floor(frac[3 * t + 1] / sy);
    py = py % ny;
    while (py < 0) py += ny;
    int pz = (int)std::floor(frac[3 * t + 2] / sz);
    pz = pz % nz;
    while (pz < 0) pz += nz;
    int c = px + py * nx + pz * (nx * ny);
    if ((int)cells[c].size() < MPC) cells[c].push_back(t);
    else status = ERR_CELL_OVERFLOW;
  }
  std::fill(howmany, howmany + N, 0);
  const T cut2 = Rc * Rc;
  for (int cz = 0; cz < nz; cz++)
    for (int cy = 0; cy < ny; cy++)
      for (int cx = 0; cx < nx; cx++) {
        const std::vector<int>& cen = cells[cx + cy * nx + cz * nx * ny];
        for (int who : cen) {
          const T* pi = frac + 3 * who;
          for (int i = -1; i < 2; i++) {
            int bi = cx + i;
            if (bi < 0) bi = nx - 1; else if (bi == nx) bi = 0;
            for (int j = -1; j < 2; j++) {
              int bj = cy + j;
              if (bj < 0) bj = ny - 1; else if (bj == ny) bj = 0;
              for (int k = -1; k < 2; k++) {
                int bk = cz + k;
                if (bk < 0) bk = nz - 1; else if (bk == nz) bk = 0;
                const std::vector<int>& nb = cells[bi + bj * nx + bk * nx * ny];
                for (int he : nb) {
                  T d[3];
                  mic(box, frac + 3 * he, pi, d);
                  T dist2 = d[0] * d[0] + d[1] * d[1] + d[2] * d[2];
                  if (dist2 < cut2 && who != he) {
                    int slot = howmany[who]++;
                    if (slot < nr) {
                      with[who * nr + slot] = he;
                      with_d2[who * nr + slot] = dist2;
                    }
                  }
                }
              }
            }
          }
        }
      }
  for (int i = 0; i < N; i++) {
    int n = howmany[i];
    if (n > nr) { status = ERR_RADIAL_OVERFLOW; n = nr; }
    int* rw = with + i * nr;
    T* rr = with_d2 + i * nr;
    for (int a = 1; a < n; ++a) {
      T kr = rr[a];
      int kw = rw[a];
      int b = a - 1;
      while (b >= 0 && rr[b] > kr) {
        rr[b + 1] = rr[b];
        rw[b + 1] = rw[b];
        --b;
      }
      rr[b + 1] = kr;
      rw[b + 1] = kw;
    }
  }
  return status;
}

// ComputeDescriptorsLight: descriptor_builder/reforce.cc:262-444 and the two
// kernels of reforce.cu.cc.  Outputs follow the op's layouts; float slots the
// reference leaves undefined are zero here.  nbr_d2 (optional) returns the sorted
// squared distances for tie analysis.
template <class T>
int descriptors(const DescCfg<T>& c, int nf, int N, const T* pos, const T* box, T* raddescr, T* angdescr,
                T* des3bsupp, int* intmap2b, int* intmap3b, T* der2b, T* der3b, T* der3bsupp, int* numtriplet,
                T* nbr_d2 /*nullable [nf,N,nr]*/) {
  const T PI = PIc<T>();
  const int nr = c.nr, na = c.na;
  std::fill(raddescr, raddescr + (size_t)nf * N * nr, T(0));
  std::fill(des3bsupp, des3bsupp + (size_t)nf * N * nr, T(0));
  std::fill(der2b, der2b + (size_t)nf * N * 3 * nr, T(0));
  std::fill(der3bsupp, der3bsupp + (size_t)nf * N * 3 * nr, T(0));
  std::fill(angdescr, angdescr + (size_t)nf * N * na, T(0));
  std::fill(der3b, der3b + (size_t)nf * N * 3 * na * 2, T(0));
  std::fill(intmap2b, intmap2b + (size_t)nf * N * (nr + 1), 0);
  std::fill(intmap3b, intmap3b + (size_t)nf * N * na * 2, 0);
  std::fill(numtriplet, numtriplet + (size_t)nf * N, 0);
  int status = OK;
  std::vector<T> frac((size_t)3 * N), d2((size_t)N * nr);
  std::vector<int> with((size_t)N * nr), howmany(N);
  for (int b = 0; b < nf; b++) {
    const T* bx = box + 6 * b;
    int st = neighbour_list(c.Rc, nr, N, pos + (size_t)b * 3 * N, bx, frac.data(), with.data(), howmany.data(),
                            d2.data(), (int*)nullptr);
    if (st != OK && status == OK) status = st;
    if (st == ERR_BAD_BOX) continue;
    if (nbr_d2) std::copy(d2.begin(), d2.end(), nbr_d2 + (size_t)b * N * nr);
#pragma omp parallel for schedule(static)
    for (int i = 0; i < N; i++) {
      int n = std::min(howmany[i], nr);
      size_t base = ((size_t)b * N + i);
      intmap2b[base * (nr + 1)] = howmany[i];
      int nang = 0;
      for (int k = 0; k < n; k++) {  // reforce.cu.cc:17-110
        int j = with[i * nr + k];
        T dist[3];
        mic(bx, frac.data() + 3 * i, frac.data() + 3 * j, dist);
        T dn = std::sqrt(dist[0] * dist[0] + dist[1] * dist[1] + dist[2] * dist[2]);
        T* d3s = der3bsupp + base * 3 * nr;
        T* d2b = der2b + base * 3 * nr;
        if (dn < c.Ra) {
          nang++;
          des3bsupp[base * nr + k] = 0.5 * (std::cos(PI * dn / c.Ra) + 1);
          for (int a = 0; a < 3; a++)
            d3s[a * nr + k] = -0.5 * std::sin(PI * dn / c.Ra) * PI / c.Ra * dist[a] / dn;
        }
        if (dn < c.Rs) {
          raddescr[base * nr + k] =
              c.coeffA / std::pow(dn, c.pow_alpha) + c.coeffB / std::pow(dn, c.pow_beta) + c.coeffC;
          for (int a = 0; a < 3; a++)
            d2b[a * nr + k] = (-c.pow_alpha * c.coeffA / std::pow(dn, c.pow_alpha + T(1.)) -
                               c.pow_beta * c.coeffB / std::pow(dn, c.pow_beta + T(1.))) *
                              dist[a] / dn;
        } else {
          raddescr[base * nr + k] = 0.5 * (std::cos(PI * dn / c.Rc) + 1);
          for (int a = 0; a < 3; a++) d2b[a * nr + k] = -0.5 * std::sin(PI * dn / c.Rc) * PI / c.Rc * dist[a] / dn;
        }
        intmap2b[base * (nr + 1) + 1 + k] = j;
      }
      numtriplet[base] = nang;
    }
    for (int i = 0; i < N; i++) {
      int m = numtriplet[(size_t)b * N + i];
      if (m * (m - 1) / 2 > na) { if (status == OK) status = ERR_ANGULAR_OVERFLOW; }
    }
#pragma omp parallel for schedule(dynamic, 8)
    for (int i = 0; i < N; i++) {  // reforce.cu.cc:112-236
      size_t base = ((size_t)b * N + i);
      int m = numtriplet[base];
      int nn = 0;
      for (int j = 0; j < m - 1; j++)
        for (int k = j + 1; k < m; k++, nn++) {
          if (nn >= na) continue;
          int jw = with[i * nr + j], kw = with[i * nr + k];
          intmap3b[(base * na + nn) * 2 + 0] = jw;
          intmap3b[(base * na + nn) * 2 + 1] = kw;
          T dj[3], dk[3];
          mic(bx, frac.data() + 3 * i, frac.data() + 3 * jw, dj);
          mic(bx, frac.data() + 3 * i, frac.data() + 3 * kw, dk);
          T nj = std::sqrt(dj[0] * dj[0] + dj[1] * dj[1] + dj[2] * dj[2]);
          T nk = std::sqrt(dk[0] * dk[0] + dk[1] * dk[1] + dk[2] * dk[2]);
          T dot = dj[0] * dk[0] + dj[1] * dk[1] + dj[2] * dk[2];
          T angle = dot / (nj * nk);
          T cj = T(0.5) * (T(1.) + std::cos(PI * nj / c.Ra));
          T ck = T(0.5) * (T(1.) + std::cos(PI * nk / c.Ra));
          T tijk = 0.5 * (angle + 1) * cj * ck;
          T* d3 = der3b + base * 3 * na * 2;
          for (int a = 0; a < 3; a++) {
            T dcij = -T(0.5) * std::sin(PI * nj / c.Ra) * PI / c.Ra / nj * dj[a];
            T dcik = -T(0.5) * std::sin(PI * nk / c.Ra) * PI / c.Ra / nk * dk[a];
            T daij = 0.5 * ((nj * nj) * dk[a] - dj[a] * dot) / (nj * nj * nj * nk);
            T daik = 0.5 * ((nk * nk) * dj[a] - dk[a] * dot) / (nk * nk * nk * nj);
            d3[((size_t)a * na + nn) * 2 + 0] = daij * cj * ck + 0.5 * (angle + 1) * dcij * ck;
            d3[((size_t)a * na + nn) * 2 + 1] = daik * cj * ck + 0.5 * (angle + 1) * cj * dcik;
          }
          angdescr[base * na + nn] = tijk;
        }
    }
  }
  return status;
}

// Unrank the triplet slot nn into the pair (j<k) of sorted-neighbour positions
// for a row of m angular neighbours: reforce.cu.cc:137-146.
inline void unrank(int nn, int m, int* jo, int* ko) {
  int j = 0, prev = 0, next = m - j - 1;
  while (nn >= next) {
    j += 1;
    prev = next;
    next += m - j - 1;
  }
  *jo = j;
  *ko = nn - prev + 1 + j;
}

// ---------------------------------------------------------------------------
// ComputeSortProj: fingerprint/rad/reforce.cu.cc:12-48.
template <class T>
void af_radial(int nf, int Nl, int nr, int Fr, const T* raddescr, const int* intmap2b, const T* alpha2b, const T* e2,
               const int* type_map, T* out) {
#pragma omp parallel for schedule(static)
  for (int bp = 0; bp < nf * Nl; bp++) {
    int n = std::min(intmap2b[(size_t)bp * (nr + 1)], nr);
    std::vector<double> acc(Fr, 0.0);
    for (int j = 0; j < n; j++) {
      T d = raddescr[(size_t)bp * nr + j];
      int tj = type_map[intmap2b[(size_t)bp * (nr + 1) + 1 + j]];
      for (int i = 0; i < Fr; i++) {
        T w = std::exp(alpha2b[Fr * tj + i] * d) * e2[Fr * tj + i];
        acc[i] += (double)(d * w);
      }
    }
    for (int i = 0; i < Fr; i++) out[(size_t)bp * Fr + i] = (T)acc[i];
  }
}

// ComputeSortProj3body: fingerprint/ang/reforce.cu.cc:13-71.  ds = des3bsupp.
template <class T>
void af_angular(int nf, int Nl, int nr, int na, int Fa, const T* angdescr, const T* ds, const int* intmap3b,
                const T* alpha3b, const T* e3, const int* type_map, const int* numtriplet, T* out) {
#pragma omp parallel for schedule(dynamic, 8)
  for (int bp = 0; bp < nf * Nl; bp++) {
    int m = numtriplet[bp];
    int nt3 = std::min(m * (m - 1) / 2, na);
    std::vector<double> acc(Fa, 0.0);
    for (int nn = 0; nn < nt3; nn++) {
      int j, k;
      unrank(nn, m, &j, &k);
      int sum = type_map[intmap3b[((size_t)bp * na + nn) * 2]] + type_map[intmap3b[((size_t)bp * na + nn) * 2 + 1]];
      T t = angdescr[(size_t)bp * na + nn];
      T dj = ds[(size_t)bp * nr + j], dk = ds[(size_t)bp * nr + k];
      for (int a = 0; a < Fa; a++) {
        T a1 = alpha3b[(sum * Fa + a) * 3], a2 = alpha3b[(sum * Fa + a) * 3 + 1], be = alpha3b[(sum * Fa + a) * 3 + 2];
        T ch = e3[sum * Fa + a];
        T sw = std::exp(a1 * dj + a2 * dk);
        sw += std::exp(a2 * dj + a1 * dk);
        sw *= std::exp(be * t);
        acc[a] += (double)(t * sw * ch / T(2.));
      }
    }
    for (int a = 0; a < Fa; a++) out[(size_t)bp * Fa + a] = (T)acc[a];
  }
}

// Minimum-image separation r_i - r_j from Cartesian positions, as the virial kernels form it
// (STAF/include/staf_force_pbc.cuh:15-49: Cartesian -> fractional with the inverse box, rint wrap, back).
template <class T>
inline void mic_cart(const T* pi, const T* pj, const T* B, T* d) {
  T I[6];
  I[0] = T(1.) / B[0];
  I[1] = -B[1] / (B[0] * B[3]);
  I[2] = (B[1] * B[4]) / (B[0] * B[3] * B[5]) - B[2] / (B[0] * B[5]);
  I[3] = T(1.) / B[3];
  I[4] = -B[4] / (B[3] * B[5]);
  I[5] = T(1.) / B[5];
  T fi[3] = {I[0] * pi[0] + I[1] * pi[1] + I[2] * pi[2], I[3] * pi[1] + I[4] * pi[2], I[5] * pi[2]};
  T fj[3] = {I[0] * pj[0] + I[1] * pj[1] + I[2] * pj[2], I[3] * pj[1] + I[4] * pj[2], I[5] * pj[2]};
  T r[3] = {fi[0] - fj[0], fi[1] - fj[1], fi[2] - fj[2]};
  for (int a = 0; a < 3; a++) r[a] -= std::rint(r[a]);
  d[0] = B[0] * r[0] + B[1] * r[1] + B[2] * r[2];
  d[1] = B[3] * r[1] + B[4] * r[2];
  d[2] = B[5] * r[2];
}

// ComputeForceRadial: force/rad/reforce.cu.cc:45-136.  force[nf,3N] is ADDED to.
template <class T>
void force_radial(int nf, int Nl, int N, int nr, int Fr, int shift, const T* netderiv, const T* der2b,
                  const int* intmap2b, const T* raddescr, const T* alpha2b, const T* e2, const int* type_map,
                  double* force /*[nf,3N] double accumulators*/, const T* pos = nullptr, const T* box = nullptr,
                  double* virial = nullptr /*[nf,9]: ComputeForceRadialVirial, force/rad/reforce.cu.cc:174-287*/) {
#pragma omp parallel for schedule(static)
  for (int bp = 0; bp < nf * Nl; bp++) {
    int b = bp / Nl, par = bp % Nl, ipar = par + shift;
    int n = std::min(intmap2b[(size_t)bp * (nr + 1)], nr);
    double fi[3] = {0, 0, 0};
    for (int j = 0; j < n; j++) {
      int nj = intmap2b[(size_t)bp * (nr + 1) + 1 + j];
      T d = raddescr[(size_t)bp * nr + j];
      int tj = type_map[nj];
      double fj[3] = {0, 0, 0};
      for (int i = 0; i < Fr; i++) {
        T al = alpha2b[Fr * tj + i], ch = e2[Fr * tj + i];
        T sds = ch * std::exp(al * d);
        sds *= (T(1.) + al * d);
        T pg = netderiv[(size_t)bp * Fr + i];
        for (int a = 0; a < 3; a++) {
          T tmp = T(0.5) * sds * der2b[((size_t)bp * 3 + a) * nr + j];
          fi[a] -= (double)(pg * tmp);
          fj[a] += (double)(pg * tmp);
        }
      }
      for (int a = 0; a < 3; a++) atomic_add(&force[((size_t)b * N + nj) * 3 + a], fj[a]);
      if (virial) {  // W_ab -= g_a r_b
        T r[3];
        mic_cart(pos + ((size_t)b * N + ipar) * 3, pos + ((size_t)b * N + nj) * 3, box + (size_t)b * 6, r);
        for (int a = 0; a < 3; a++)
          for (int c = 0; c < 3; c++) atomic_add(&virial[(size_t)b * 9 + a * 3 + c], -fj[a] * (double)r[c]);
      }
    }
    for (int a = 0; a < 3; a++) atomic_add(&force[((size_t)b * N + ipar) * 3 + a], fi[a]);
  }
}

// ComputeForceTripl: force/ang/reforce.cu.cc:48-232; with pos/box/virial the ...Virial variant (:269-457).
template <class T>
void force_tripl(int nf, int Nl, int N, int nr, int na, int Fa, int shift, const T* netderiv, const T* ds,
                 const T* angdescr, const T* der3bsupp, const T* der3b, const int* intmap3b, const T* alpha3b,
                 const T* e3, const int* type_map, const int* numtriplet, double* force, const T* pos = nullptr,
                 const T* box = nullptr, double* virial = nullptr) {
#pragma omp parallel for schedule(dynamic, 8)
  for (int bp = 0; bp < nf * Nl; bp++) {
    int b = bp / Nl, par = bp % Nl, ipar = par + shift;
    int m = numtriplet[bp];
    int nt3 = std::min(m * (m - 1) / 2, na);
    double fi[3] = {0, 0, 0};
    for (int nn = 0; nn < nt3; nn++) {
      double fj[3] = {0, 0, 0}, fk[3] = {0, 0, 0};
      int j, k;
      unrank(nn, m, &j, &k);
      int nj = intmap3b[((size_t)bp * na + nn) * 2], nk = intmap3b[((size_t)bp * na + nn) * 2 + 1];
      int sum = type_map[nj] + type_map[nk];
      T t = angdescr[(size_t)bp * na + nn];
      T rj = ds[(size_t)bp * nr + j], rk = ds[(size_t)bp * nr + k];
      for (int a1 = 0; a1 < Fa; a1++) {
        T ax = alpha3b[(sum * Fa + a1) * 3], ay = alpha3b[(sum * Fa + a1) * 3 + 1], az = alpha3b[(sum * Fa + a1) * 3 + 2];
        T ch = e3[sum * Fa + a1];
        T nd = T(0.5) * netderiv[(size_t)bp * Fa + a1] * ch;
        T eb = std::exp(az * t);
        T sim1 = std::exp(ay * rj + ax * rk);
        T sim2 = std::exp(ax * rj + ay * rk);
        T delta = eb * (1. + az * t) * (sim1 + sim2) * T(0.5);
        T suppj = (ax * sim2 + ay * sim1) * eb * T(0.5);
        T suppk = (ax * sim1 + ay * sim2) * eb * T(0.5);
        T Bj = suppj * t, Bk = suppk * t;
        for (int a = 0; a < 3; a++) {
          T ix = der3b[(((size_t)bp * 3 + a) * na + nn) * 2], iy = der3b[(((size_t)bp * 3 + a) * na + nn) * 2 + 1];
          T irj = der3bsupp[((size_t)bp * 3 + a) * nr + j], irk = der3bsupp[((size_t)bp * 3 + a) * nr + k];
          T fij = nd * (delta * ix + Bj * irj);
          T fik = nd * (delta * iy + Bk * irk);
          fi[a] -= (double)(fij + fik);
          fj[a] += (double)fij;
          fk[a] += (double)fik;
        }
      }
      for (int a = 0; a < 3; a++) {
        atomic_add(&force[((size_t)b * N + nj) * 3 + a], fj[a]);
        atomic_add(&force[((size_t)b * N + nk) * 3 + a], fk[a]);
      }
      if (virial) {  // W_ab -= f_ij,a r_ij,b + f_ik,a r_ik,b
        T rij[3], rik[3];
        mic_cart(pos + ((size_t)b * N + ipar) * 3, pos + ((size_t)b * N + nj) * 3, box + (size_t)b * 6, rij);
        mic_cart(pos + ((size_t)b * N + ipar) * 3, pos + ((size_t)b * N + nk) * 3, box + (size_t)b * 6, rik);
        for (int a = 0; a < 3; a++)
          for (int c = 0; c < 3; c++)
            atomic_add(&virial[(size_t)b * 9 + a * 3 + c], -(fj[a] * (double)rij[c] + fk[a] * (double)rik[c]));
      }
    }
    for (int a = 0; a < 3; a++) atomic_add(&force[((size_t)b * N + ipar) * 3 + a], fi[a]);
  }
}

// ComputeTwoBodyParGrad: grad_finger/rad/reforce.cu.cc:12-46.
template <class T>
void grad_af_radial(int nf, int Nl, int nr, int Fr, int nt, const T* prevgrad, const T* raddescr, const int* intmap2b,
                    const T* alpha2b, const T* e2, const int* type_map, double* g_alpha /*[nt,Fr]*/,
                    double* g_emb /*[nt,Fr]*/) {
  ThreadAcc ta((size_t)2 * nt * Fr);
#pragma omp parallel for schedule(static)
  for (int bp = 0; bp < nf * Nl; bp++) {
    double* ga = ta.mine();
    double* ge = ga + nt * Fr;
    int n = std::min(intmap2b[(size_t)bp * (nr + 1)], nr);
    for (int j = 0; j < n; j++) {
      T d = raddescr[(size_t)bp * nr + j];
      int cht = type_map[intmap2b[(size_t)bp * (nr + 1) + 1 + j]];
      for (int i = 0; i < Fr; i++) {
        T pg = prevgrad[(size_t)bp * Fr + i];
        T tw = e2[cht * Fr + i];
        T acc = d * d;
        acc *= std::exp(alpha2b[cht * Fr + i] * d) * tw * pg;
        ga[cht * Fr + i] += (double)acc;
        acc = d;
        acc *= std::exp(alpha2b[cht * Fr + i] * d) * pg;
        ge[cht * Fr + i] += (double)acc;
      }
    }
  }
  std::vector<double> tot((size_t)2 * nt * Fr, 0.0);
  ta.merge_into(tot.data());
  for (int i = 0; i < nt * Fr; i++) { g_alpha[i] += tot[i]; g_emb[i] += tot[nt * Fr + i]; }
}

// ComputeSortProj3bodyGrad: grad_finger/ang/reforce.cu.cc:13-111.  The second
// output of the op (emb3b gradient) is never written by the reference: zeros.
template <class T>
void grad_af_angular(int nf, int Nl, int nr, int na, int Fa, const T* prevgrad, const T* angdescr, const T* ds,
                     const int* intmap3b, const T* alpha3b, const T* e3, const int* type_map, const int* numtriplet,
                     int C, double* g_alpha3_out /*[C,3Fa]*/) {
  ThreadAcc ta((size_t)C * 3 * Fa);
#pragma omp parallel for schedule(dynamic, 8)
  for (int bp = 0; bp < nf * Nl; bp++) {
    double* g_alpha3 = ta.mine();
    int m = numtriplet[bp];
    int nt3 = std::min(m * (m - 1) / 2, na);
    for (int nn = 0; nn < nt3; nn++) {
      int j, k;
      unrank(nn, m, &j, &k);
      int sum = type_map[intmap3b[((size_t)bp * na + nn) * 2]] + type_map[intmap3b[((size_t)bp * na + nn) * 2 + 1]];
      T Tjy = angdescr[(size_t)bp * na + nn];
      T dj = ds[(size_t)bp * nr + j], dy = ds[(size_t)bp * nr + k];
      for (int a1 = 0; a1 < Fa; a1++) {
        T al1 = alpha3b[(sum * Fa + a1) * 3], al2 = alpha3b[(sum * Fa + a1) * 3 + 1], be = alpha3b[(sum * Fa + a1) * 3 + 2];
        T ch = e3[sum * Fa + a1];
        T pg = prevgrad[(size_t)bp * Fa + a1];
        T e12 = std::exp(al1 * dj + al2 * dy);
        T e21 = std::exp(al1 * dy + al2 * dj);
        T bt = std::exp(be * Tjy);
        g_alpha3[(sum * Fa + a1) * 3 + 0] += (double)(pg * ch * (e12 * dj + e21 * dy) * bt * Tjy / T(2.));
        g_alpha3[(sum * Fa + a1) * 3 + 1] += (double)(pg * ch * (e12 * dy + e21 * dj) * bt * Tjy / T(2.));
        g_alpha3[(sum * Fa + a1) * 3 + 2] += (double)(pg * ch * (e12 + e21) * bt * Tjy * Tjy / T(2.));
      }
    }
  }
  ta.merge_into(g_alpha3_out);
}

// ComputeForceRadialGrad: grad_force/rad/reforce.cu.cc:46-123.
template <class T>
void grad_force_radial(int nf, int Nl, int N, int nr, int Fr, int shift, const T* prevgrad /*[nf,3N]*/,
                       const T* netderiv, const T* der2b, const int* intmap2b, const T* raddescr, const T* alpha2b,
                       const T* e2, const int* type_map, int nt, double* gradnet /*[nf,Nl,Fr]*/,
                       double* g_alpha_out, double* g_emb_out, const T* pos = nullptr, const T* box = nullptr,
                       const T* wbar = nullptr /*[nf,9] dL/dvirial: ...VirialGrad, grad_force/rad/reforce.cu.cc:165-234*/) {
  ThreadAcc ta((size_t)2 * nt * Fr);
#pragma omp parallel for schedule(static)
  for (int bp = 0; bp < nf * Nl; bp++) {
    double* g_alpha = ta.mine();
    double* g_emb = g_alpha + nt * Fr;
    int b = bp / Nl, par = bp % Nl, ipar = par + shift;
    int n = std::min(intmap2b[(size_t)bp * (nr + 1)], nr);
    for (int j = 0; j < n; j++) {
      int nj = intmap2b[(size_t)bp * (nr + 1) + 1 + j];
      int cht = type_map[nj];
      T d = raddescr[(size_t)bp * nr + j];
      T wdot[3] = {0, 0, 0};  // (dL/dW r)_a: the virial cotangent acts like a shift of the neighbour's force cotangent
      if (wbar) {
        T r[3];
        mic_cart(pos + ((size_t)b * N + ipar) * 3, pos + ((size_t)b * N + nj) * 3, box + (size_t)b * 6, r);
        const T* Wg = wbar + (size_t)b * 9;
        for (int a = 0; a < 3; a++) wdot[a] = Wg[a * 3] * r[0] + Wg[a * 3 + 1] * r[1] + Wg[a * 3 + 2] * r[2];
      }
      for (int i = 0; i < Fr; i++) {
        T a1 = 0, a2 = 0, a3 = 0;
        for (int a = 0; a < 3; a++) {
          T pe = prevgrad[((size_t)b * N + ipar) * 3 + a], pn = prevgrad[((size_t)b * N + nj) * 3 + a] - wdot[a];
          T common = T(0.5) * der2b[((size_t)bp * 3 + a) * nr + j];
          T al = alpha2b[Fr * cht + i], ch = e2[Fr * cht + i];
          T s1 = std::exp(al * d);
          T sds = s1 * (T(1.) + al * d);
          T ba = ch * s1 * d * (T(2.) + al * d);
          T NG = netderiv[(size_t)bp * Fr + i];
          a1 -= pe * common * ch * sds;
          a1 += pn * common * ch * sds;
          a2 -= pe * NG * ba * common;
          a2 += pn * NG * ba * common;
          a3 -= pe * NG * sds * common;
          a3 += pn * NG * sds * common;
        }
        gradnet[(size_t)bp * Fr + i] += (double)a1;
        g_alpha[Fr * cht + i] += (double)a2;
        g_emb[Fr * cht + i] += (double)a3;
      }
    }
  }
  std::vector<double> tot((size_t)2 * nt * Fr, 0.0);
  ta.merge_into(tot.data());
  for (int i = 0; i < nt * Fr; i++) { g_alpha_out[i] += tot[i]; g_emb_out[i] += tot[nt * Fr + i]; }
}

// ComputeForceTriplGrad: grad_force/ang/reforce.cu.cc:47-231.  The third output
// of the op (gradck) is never written by the reference: zeros.
template <class T>
void grad_force_tripl(int nf, int Nl, int N, int nr, int na, int Fa, int shift, const T* prevgrad, const T* netderiv,
                      const T* ds, const T* angdescr, const T* der3bsupp, const T* der3b, const int* intmap3b,
                      const T* alpha3b, const T* e3, const int* type_map, const int* numtriplet, int C,
                      double* gradnet /*[nf,Nl,Fa]*/, double* g_alpha3_out /*[C,3Fa]*/, const T* pos = nullptr,
                      const T* box = nullptr, const T* wbar = nullptr /*grad_force/ang/reforce.cu.cc:274-446*/) {
  ThreadAcc ta((size_t)C * 3 * Fa);
#pragma omp parallel for schedule(dynamic, 8)
  for (int bp = 0; bp < nf * Nl; bp++) {
    double* g_alpha3 = ta.mine();
    int b = bp / Nl, par = bp % Nl, ipar = par + shift;
    int m = numtriplet[bp];
    int nt3 = std::min(m * (m - 1) / 2, na);
    for (int nn = 0; nn < nt3; nn++) {
      int j, k;
      unrank(nn, m, &j, &k);
      int nj = intmap3b[((size_t)bp * na + nn) * 2], nk = intmap3b[((size_t)bp * na + nn) * 2 + 1];
      int sum = type_map[nj] + type_map[nk];
      T t = angdescr[(size_t)bp * na + nn];
      T rj = ds[(size_t)bp * nr + j], rk = ds[(size_t)bp * nr + k];
      T wij[3] = {0, 0, 0}, wik[3] = {0, 0, 0};
      if (wbar) {
        T rij[3], rik[3];
        mic_cart(pos + ((size_t)b * N + ipar) * 3, pos + ((size_t)b * N + nj) * 3, box + (size_t)b * 6, rij);
        mic_cart(pos + ((size_t)b * N + ipar) * 3, pos + ((size_t)b * N + nk) * 3, box + (size_t)b * 6, rik);
        const T* Wg = wbar + (size_t)b * 9;
        for (int a = 0; a < 3; a++) {
          wij[a] = Wg[a * 3] * rij[0] + Wg[a * 3 + 1] * rij[1] + Wg[a * 3 + 2] * rij[2];
          wik[a] = Wg[a * 3] * rik[0] + Wg[a * 3 + 1] * rik[1] + Wg[a * 3 + 2] * rik[2];
        }
      }
      for (int c = 0; c < Fa; c++) {
        T NG = netderiv[(size_t)bp * Fa + c];
        T ax = alpha3b[(sum * Fa + c) * 3], ay = alpha3b[(sum * Fa + c) * 3 + 1], az = alpha3b[(sum * Fa + c) * 3 + 2];
        T ch = e3[sum * Fa + c];
        T eb = std::exp(az * t);
        T sim1 = std::exp(ay * rj + ax * rk);
        T sim2 = std::exp(ax * rj + ay * rk);
        T ss = sim1 + sim2;
        T delta = eb * (T(1.0) + az * t) * ss * T(0.5);
        T suppj = (ax * sim2 + ay * sim1) * eb;
        T suppk = (ax * sim1 + ay * sim2) * eb;
        T Bj = suppj * t * T(0.5), Bk = suppk * t * T(0.5);
        T acc1 = 0, acc3 = 0, acc4 = 0, acc5 = 0;
        for (int cor = 0; cor < 3; cor++) {
          T ix = der3b[(((size_t)bp * 3 + cor) * na + nn) * 2], iy = der3b[(((size_t)bp * 3 + cor) * na + nn) * 2 + 1];
          T irj = der3bsupp[((size_t)bp * 3 + cor) * nr + j], irk = der3bsupp[((size_t)bp * 3 + cor) * nr + k];
          T pl = prevgrad[((size_t)b * N + ipar) * 3 + cor];
          T pj = prevgrad[((size_t)b * N + nj) * 3 + cor] - wij[cor], pk = prevgrad[((size_t)b * N + nk) * 3 + cor] - wik[cor];
          T gij = ch * delta * ix + ch * Bj * irj;
          T gik = ch * delta * iy + ch * Bk * irk;
          acc1 += -pl * T(0.5) * (gij + gik);
          acc1 += pj * T(0.5) * gij + pk * T(0.5) * gik;
          T ba1 = eb * (T(1.) + az * t) * (sim1 * rk + sim2 * rj) * T(0.5);
          T ba2 = eb * (T(1.) + az * t) * (sim1 * rj + sim2 * rk) * T(0.5);
          T bb = eb * t * (T(2.) + az * t) * ss * T(0.5);
          T bbj = suppj * t * t * T(0.5), bbk = suppk * t * t * T(0.5);
          T a1j = (sim2 + ax * sim2 * rj + ay * sim1 * rk) * eb * T(0.5) * t;
          T a2j = (sim1 + ay * sim1 * rj + ax * sim2 * rk) * eb * T(0.5) * t;
          T a1k = (sim1 + ax * sim1 * rk + ay * sim2 * rj) * eb * T(0.5) * t;
          T a2k = (sim2 + ay * sim2 * rk + ax * sim1 * rj) * eb * T(0.5) * t;
          T g1ij = ch * ba1 * ix + ch * a1j * irj, g1ik = ch * ba1 * iy + ch * a1k * irk;
          T g2ij = ch * ba2 * ix + ch * a2j * irj, g2ik = ch * ba2 * iy + ch * a2k * irk;
          T gbij = ch * bb * ix + ch * bbj * irj, gbik = ch * bb * iy + ch * bbk * irk;
          acc3 += -pl * T(0.5) * NG * (g1ij + g1ik) + pj * T(0.5) * NG * g1ij + pk * T(0.5) * NG * g1ik;
          acc4 += -pl * T(0.5) * NG * (g2ij + g2ik) + pj * T(0.5) * NG * g2ij + pk * T(0.5) * NG * g2ik;
          acc5 += -pl * T(0.5) * NG * (gbij + gbik) + pj * T(0.5) * NG * gbij + pk * T(0.5) * NG * gbik;
        }
        gradnet[(size_t)bp * Fa + c] += (double)acc1;
        g_alpha3[(sum * Fa + c) * 3 + 0] += (double)acc3;
        g_alpha3[(sum * Fa + c) * 3 + 1] += (double)acc4;
        g_alpha3[(sum * Fa + c) * 3 + 2] += (double)acc5;
      }
    }
  }
  ta.merge_into(g_alpha3_out);
}

// ---------------------------------------------------------------------------
// Per-species MLP head.  x = log(AF + 1e-3) - mu; Dense(tanh) ... Dense(1).
// Weights row-major [in,out] as Keras (staf_mlp_ort.cc:20-24).
struct MlpShape {
  int n_in;
  int n_dense;            // number of Dense layers including the output layer
  int width[MAX_DENSE];   // output width of each Dense; width[n_dense-1] == 1
  int in_of(int l) const { return l == 0 ? n_in : width[l - 1]; }
  int n_weights() const {
    int s = 0;
    for (int l = 0; l < n_dense; l++) s += in_of(l) * width[l] + width[l];
    return s;
  }
  int w_off(int l) const {
    int s = 0;
    for (int k = 0; k < l; k++) s += in_of(k) * width[k] + width[k];
    return s;
  }
  int b_off(int l) const { return w_off(l) + in_of(l) * width[l]; }
};

// Forward + d(sum e)/dAF (staf_model.py:188-191; staf_mlp_ort.cc:196-242), and,
// when ebar/u are given, the backward of  S = sum_a ebar[a]*e[a] + sum_{a,c} u[a,c]*netderiv[a,c]
// with respect to the weights, mu and AF (what tf.gradients does through
// grad_ene for the force loss: staf_model.py:225-228).
template <class T>
void mlp_eval(const MlpShape& sh, int n_atoms, const T* af, const T* mu, const T* w /*packed*/, T* e_out,
              T* netderiv_out, const T* ebar /*nullable [n]*/, const T* u /*nullable [n,F]*/,
              double* g_w /*[n_weights]*/, double* g_mu /*[F]*/, T* g_af /*[n,F]*/) {
  const int F = sh.n_in, L = sh.n_dense;
  int maxw = F;
  for (int l = 0; l < L; l++) maxw = std::max(maxw, sh.width[l]);
  const bool bwd = (g_w != nullptr);
  int nth = 1;
#ifdef _OPENMP
  nth = omp_get_max_threads();
#endif
  std::vector<std::vector<double>> gw_t(bwd ? nth : 0), gmu_t(bwd ? nth : 0);
  for (auto& v : gw_t) v.assign(sh.n_weights(), 0.0);
  for (auto& v : gmu_t) v.assign(F, 0.0);
#pragma omp parallel
  {
    int tid = 0;
#ifdef _OPENMP
    tid = omp_get_thread_num();
#endif
    std::vector<std::vector<T>> h(L + 1), hd(L + 1), P(L + 1), Q(L + 1);
    for (int l = 0; l <= L; l++) {
      int wdt = (l == 0) ? F : sh.width[l - 1];
      h[l].assign(wdt, 0);
      hd[l].assign(wdt, 0);
      P[l].assign(wdt, 0);
      Q[l].assign(wdt, 0);
    }
    std::vector<T> delta(maxw), delta2(maxw), v(F);
#pragma omp for schedule(static)
    for (int a = 0; a < n_atoms; a++) {
      const T* afa = af + (size_t)a * F;
      for (int i = 0; i < F; i++) h[0][i] = std::log(afa[i] + T(1e-3)) - mu[i];
      for (int l = 0; l < L; l++) {
        int in = sh.in_of(l), out = sh.width[l];
        const T* W = w + sh.w_off(l);
        const T* B = w + sh.b_off(l);
        for (int j = 0; j < out; j++) {
          T s = B[j];
          for (int i = 0; i < in; i++) s += h[l][i] * W[i * out + j];
          if (l < L - 1) s = std::tanh(s);
          h[l + 1][j] = s;
        }
      }
      if (e_out) e_out[a] = h[L][0];
      // reverse sweep for de/dx: delta at layer output, including activation derivative
      // P[l] = de/d(pre-activation input vector of layer l) ... stored as de/dh[l]
      P[L][0] = T(1);
      for (int l = L - 1; l >= 0; l--) {
        int in = sh.in_of(l), out = sh.width[l];
        const T* W = w + sh.w_off(l);
        for (int j = 0; j < out; j++) {
          T g = P[l + 1][j];
          if (l < L - 1) g *= (T(1) - h[l + 1][j] * h[l + 1][j]);
          delta[j] = g;  // de/da_l (pre-activation)
        }
        for (int i = 0; i < in; i++) {
          T s = 0;
          for (int j = 0; j < out; j++) s += delta[j] * W[i * out + j];
          P[l][i] = s;
        }
      }
      // P[0] = de/dx
      if (netderiv_out)
        for (int i = 0; i < F; i++) netderiv_out[(size_t)a * F + i] = P[0][i] / (afa[i] + T(1e-3));
      if (!bwd) continue;
      double* GW = gw_t[tid].data();
      double* GMU = gmu_t[tid].data();
      T eb = ebar ? ebar[a] : T(0);
      // (1) first-order part: eb * de/dtheta, eb * de/dAF
      //     de/dW_l[i,j] = h[l][i] * delta_l[j], recompute delta_l going down.
      // (2) second-order part: tangent v = u/(AF+eps) pushed forward, then reversed.
      for (int i = 0; i < F; i++) v[i] = u ? u[(size_t)a * F + i] / (afa[i] + T(1e-3)) : T(0);
      // forward tangent: hd[l] = d h[l] along v
      for (int i = 0; i < F; i++) hd[0][i] = v[i];
      for (int l = 0; l < L; l++) {
        int in = sh.in_of(l), out = sh.width[l];
        const T* W = w + sh.w_off(l);
        for (int j = 0; j < out; j++) {
          T s = 0;
          for (int i = 0; i < in; i++) s += hd[l][i] * W[i * out + j];
          if (l < L - 1) s *= (T(1) - h[l + 1][j] * h[l + 1][j]);
          hd[l + 1][j] = s;  // for hidden layers: d1 * adot ; for output: adot
        }
      }
      // Reverse over the pair (h, hd).  Let Sd = hd[L][0] (second-order scalar) and
      // Se = eb*h[L][0].  Cotangents: Ph[l] on h[l], Pd[l] on hd[l].
      std::vector<T>& Ph = Q[L];
      (void)Ph;
      // use Q[l] for cotangent on h[l], P[l] reused for cotangent on hd[l]
      Q[L][0] = eb;
      P[L][0] = T(1);
      for (int l = L - 1; l >= 0; l--) {
        int in = sh.in_of(l), out = sh.width[l];
        const T* W = w + sh.w_off(l);
        double* gW = GW + sh.w_off(l);
        double* gB = GW + sh.b_off(l);
        // h[l+1] = act(a), hd[l+1] = act'(a) * adot, a = h[l]W+b, adot = hd[l]W
        for (int j = 0; j < out; j++) {
          T qa, pa;  // cotangent on a and on adot
          if (l < L - 1) {
            T hh = h[l + 1][j];
            T d1 = T(1) - hh * hh;
            // adot = hd[l+1]/d1 is needed: recompute directly
            T adot = 0;
            for (int i = 0; i < in; i++) adot += hd[l][i] * W[i * out + j];
            pa = P[l + 1][j] * d1;
            // d(hd)/da = act''(a)*adot = -2*h*d1*adot ; d(h)/da = d1
            qa = Q[l + 1][j] * d1 + P[l + 1][j] * (T(-2) * hh * d1 * adot);
          } else {
            pa = P[l + 1][j];
            qa = Q[l + 1][j];
          }
          delta[j] = qa;
          delta2[j] = pa;
        }
        for (int i = 0; i < in; i++) {
          T sq = 0, sp = 0;
          for (int j = 0; j < out; j++) {
            gW[i * out + j] += (double)(h[l][i] * delta[j] + hd[l][i] * delta2[j]);
            sq += delta[j] * W[i * out + j];
            sp += delta2[j] * W[i * out + j];
          }
          Q[l][i] = sq;
          P[l][i] = sp;
        }
        for (int j = 0; j < out; j++) gB[j] += (double)delta[j];
      }
      // Q[0] = dS/dx, P[0] = dS/dv
      for (int i = 0; i < F; i++) {
        T den = afa[i] + T(1e-3);
        GMU[i] += (double)(-Q[0][i]);
        T g = Q[0][i] / den;
        if (u) g += P[0][i] * (-u[(size_t)a * F + i] / (den * den));
        if (g_af) g_af[(size_t)a * F + i] = g;
      }
    }
  }
  if (bwd) {
    for (int t = 0; t < nth; t++) {
      for (int i = 0; i < sh.n_weights(); i++) g_w[i] += gw_t[t][i];
      for (int i = 0; i < F; i++) g_mu[i] += gmu_t[t][i];
    }
  }
}

// ---------------------------------------------------------------------------
// Whole model: parameter layout shared with the GPU library's flat buffers.
struct ModelShape {
  int nt;
  int tipos[MAX_TYPES];
  int Fr[MAX_TYPES], Fa[MAX_TYPES];
  int n_dense;
  int width[MAX_DENSE];
  int C() const { return nt * (nt + 1) / 2; }
  int N() const { int s = 0; for (int t = 0; t < nt; t++) s += tipos[t]; return s; }
  int shift(int t) const { int s = 0; for (int u = 0; u < t; u++) s += tipos[u]; return s; }
  MlpShape mlp(int t) const {
    MlpShape m;
    m.n_in = Fr[t] + Fa[t];
    m.n_dense = n_dense;
    for (int l = 0; l < n_dense; l++) m.width[l] = width[l];
    return m;
  }
  // per species block: alpha2b[nt*Fr] | alpha3b[C*3*Fa] | mu[Fr+Fa] | mlp weights
  int block_size(int t) const { return nt * Fr[t] + C() * 3 * Fa[t] + Fr[t] + Fa[t] + mlp(t).n_weights(); }
  int block_off(int t) const { int s = 0; for (int u = 0; u < t; u++) s += block_size(u); return s; }
  int off_a2(int t) const { return block_off(t); }
  int off_a3(int t) const { return off_a2(t) + nt * Fr[t]; }
  int off_mu(int t) const { return off_a3(t) + C() * 3 * Fa[t]; }
  int off_w(int t) const { return off_mu(t) + Fr[t] + Fa[t]; }
  int n_params() const { return block_off(nt); }
  // squared embeddings (not trained): e2[nt*Fr] | e3[C*Fa] per species
  int emb_size(int t) const { return nt * Fr[t] + C() * Fa[t]; }
  int emb_off(int t) const { int s = 0; for (int u = 0; u < t; u++) s += emb_size(u); return s; }
  int n_emb() const { return emb_off(nt); }
};

template <class T>
inline T huber(T e) { T a = std::fabs(e); return a <= T(1) ? T(0.5) * e * e : a - T(0.5); }
template <class T>
inline T huber_d(T e) { return e > T(1) ? T(1) : (e < T(-1) ? T(-1) : e); }

// Gather the slice of atoms [shift, shift+Nl) of a [nf,N,row] tensor into [nf,Nl,row]
// (what tf.split(..., axis=1) does: staf_model.py:174-182).
template <class U>
void split_atoms(int nf, int N, int shift, int Nl, size_t row, const U* src, std::vector<U>& dst) {
  dst.resize((size_t)nf * Nl * row);
  for (int b = 0; b < nf; b++)
    std::memcpy(dst.data() + (size_t)b * Nl * row, src + ((size_t)b * N + shift) * row, sizeof(U) * Nl * row);
}

struct StepOut {
  double loss, loss_e, loss_bound, loss_f, loss_v;
};

// One energy+force evaluation, optionally with the loss and the gradient with
// respect to every trained parameter (staf_model.py:168-258, without the Adam
// update).  energy[b] = 0.5*mean_i e_i when per_atom_energy, else 0.5*sum_i e_i
// (staf_model_inference_full.py:118-119).  With v_label the loss also has the virial term of
// full_train_e_f_v (staf_model.py:313-384): pv * L(W - W_label), mean over [nf,9], W from the ...Virial force
// operators; virial_out[nf,9] receives W.
template <class T>
int energy_force_grad(const DescCfg<T>& c, const ModelShape& ms, int nf, const T* pos, const T* box,
                      const int* type_map, const T* theta, const T* emb, bool per_atom_energy, T* energy /*[nf]*/,
                      T* force /*[nf,3N]*/, bool with_grad, const T* e_label, const T* f_label, T pe, T pf, T pb,
                      T alpha_bound, int loss_kind /*0 huber, 1 mse*/, StepOut* so, T* grad /*[n_params]*/,
                      const T* v_label = nullptr /*[nf,9]*/, T pv = T(0), T* virial_out = nullptr) {
  const int N = ms.N(), nr = c.nr, na = c.na, nt = ms.nt, C = ms.C();
  size_t A = (size_t)nf * N;
  std::vector<T> rad(A * nr), ang(A * na), d3s(A * nr), der2b(A * 3 * nr), der3b(A * 3 * na * 2), der3bs(A * 3 * nr);
  std::vector<int> im2(A * (nr + 1)), im3(A * na * 2), ntr(A);
  int st = descriptors(c, nf, N, pos, box, rad.data(), ang.data(), d3s.data(), im2.data(), im3.data(), der2b.data(),
                       der3b.data(), der3bs.data(), ntr.data(), (T*)nullptr);
  if (st != OK) return st;
  struct Sp {
    std::vector<T> rad, ang, d3s, der2b, der3b, der3bs, af, e, nd;
    std::vector<int> im2, im3, ntr;
  };
  std::vector<Sp> sp(nt);
  std::vector<double> F64((size_t)nf * 3 * N, 0.0);
  std::vector<double> esum(nf, 0.0);
  const bool with_virial = v_label != nullptr || virial_out != nullptr;
  std::vector<double> W64((size_t)nf * 9, 0.0);
  const T* vpos = with_virial ? pos : nullptr;
  const T* vbox = with_virial ? box : nullptr;
  double* vW = with_virial ? W64.data() : nullptr;
  for (int t = 0; t < nt; t++) {
    Sp& s = sp[t];
    int Nl = ms.tipos[t], sh = ms.shift(t), Fr = ms.Fr[t], Fa = ms.Fa[t], F = Fr + Fa;
    split_atoms(nf, N, sh, Nl, (size_t)nr, rad.data(), s.rad);
    split_atoms(nf, N, sh, Nl, (size_t)na, ang.data(), s.ang);
    split_atoms(nf, N, sh, Nl, (size_t)nr, d3s.data(), s.d3s);
    split_atoms(nf, N, sh, Nl, (size_t)3 * nr, der2b.data(), s.der2b);
    split_atoms(nf, N, sh, Nl, (size_t)3 * na * 2, der3b.data(), s.der3b);
    split_atoms(nf, N, sh, Nl, (size_t)3 * nr, der3bs.data(), s.der3bs);
    split_atoms(nf, N, sh, Nl, (size_t)(nr + 1), im2.data(), s.im2);
    split_atoms(nf, N, sh, Nl, (size_t)na * 2, im3.data(), s.im3);
    split_atoms(nf, N, sh, Nl, (size_t)1, ntr.data(), s.ntr);
    const T* a2 = theta + ms.off_a2(t);
    const T* a3 = theta + ms.off_a3(t);
    const T* mu = theta + ms.off_mu(t);
    const T* w = theta + ms.off_w(t);
    const T* e2 = emb + ms.emb_off(t);
    const T* e3 = e2 + nt * Fr;
    size_t n = (size_t)nf * Nl;
    std::vector<T> af2(n * Fr), af3(n * Fa);
    af_radial(nf, Nl, nr, Fr, s.rad.data(), s.im2.data(), a2, e2, type_map, af2.data());
    af_angular(nf, Nl, nr, na, Fa, s.ang.data(), s.d3s.data(), s.im3.data(), a3, e3, type_map, s.ntr.data(), af3.data());
    s.af.resize(n * F);
    for (size_t a = 0; a < n; a++) {
      for (int i = 0; i < Fr; i++) s.af[a * F + i] = af2[a * Fr + i];
      for (int i = 0; i < Fa; i++) s.af[a * F + Fr + i] = af3[a * Fa + i];
    }
    s.e.resize(n);
    s.nd.resize(n * F);
    mlp_eval<T>(ms.mlp(t), (int)n, s.af.data(), mu, w, s.e.data(), s.nd.data(), nullptr, nullptr, nullptr, nullptr,
                nullptr);
    for (size_t a = 0; a < n; a++) esum[a / Nl] += (double)s.e[a];
    std::vector<T> ndr(n * Fr), nda(n * Fa);
    for (size_t a = 0; a < n; a++) {
      for (int i = 0; i < Fr; i++) ndr[a * Fr + i] = s.nd[a * F + i];
      for (int i = 0; i < Fa; i++) nda[a * Fa + i] = s.nd[a * F + Fr + i];
    }
    force_radial(nf, Nl, N, nr, Fr, sh, ndr.data(), s.der2b.data(), s.im2.data(), s.rad.data(), a2, e2, type_map,
                 F64.data(), vpos, vbox, vW);
    force_tripl(nf, Nl, N, nr, na, Fa, sh, nda.data(), s.d3s.data(), s.ang.data(), s.der3bs.data(), s.der3b.data(),
                s.im3.data(), a3, e3, type_map, s.ntr.data(), F64.data(), vpos, vbox, vW);
  }
  std::vector<T> Wv((size_t)nf * 9);
  for (size_t i = 0; i < Wv.size(); i++) Wv[i] = (T)W64[i];
  if (virial_out) std::copy(Wv.begin(), Wv.end(), virial_out);
  std::vector<T> Fv((size_t)nf * 3 * N);
  for (size_t i = 0; i < Fv.size(); i++) Fv[i] = (T)F64[i];
  if (force) std::copy(Fv.begin(), Fv.end(), force);
  std::vector<T> E(nf);
  for (int b = 0; b < nf; b++) E[b] = (T)(per_atom_energy ? 0.5 * esum[b] / N : 0.5 * esum[b]);
  if (energy) std::copy(E.begin(), E.end(), energy);
  if (!with_grad) return OK;

  // loss (staf_model.py:213-221; Keras Huber delta=1 / MSE, mean reduction)
  double le = 0, lf = 0, lb = 0;
  std::vector<T> Ebar(nf), Fbar((size_t)nf * 3 * N);
  for (int b = 0; b < nf; b++) {
    T e = E[b] - e_label[b];
    le += (double)(loss_kind == 0 ? huber(e) : e * e);
    Ebar[b] = pe * (loss_kind == 0 ? huber_d(e) : T(2) * e) / T(nf);
  }
  le /= nf;
  for (size_t i = 0; i < Fv.size(); i++) {
    T e = Fv[i] - f_label[i];
    lf += (double)(loss_kind == 0 ? huber(e) : e * e);
    Fbar[i] = pf * (loss_kind == 0 ? huber_d(e) : T(2) * e) / T((double)Fv.size());
  }
  lf /= (double)Fv.size();
  double lv = 0;
  std::vector<T> Wbar((size_t)nf * 9, T(0));
  if (v_label) {
    for (size_t i = 0; i < Wv.size(); i++) {
      T e = Wv[i] - v_label[i];
      lv += (double)(loss_kind == 0 ? huber(e) : e * e);
      Wbar[i] = pv * (loss_kind == 0 ? huber_d(e) : T(2) * e) / T((double)Wv.size());
    }
    lv /= (double)Wv.size();
  }
  const T* wb = v_label ? Wbar.data() : nullptr;
  const T* wpos = v_label ? pos : nullptr;
  const T* wbox = v_label ? box : nullptr;
  const int P = ms.n_params();
  std::vector<double> G(P, 0.0);
  for (int t = 0; t < nt; t++) {
    // bound loss: sum x*[x > bound] over alpha2b and alpha3b (staf_model.py:60-62,215-219)
    int n2 = nt * ms.Fr[t], n3 = C * 3 * ms.Fa[t];
    for (int i = 0; i < n2; i++) {
      T x = theta[ms.off_a2(t) + i];
      if (x > alpha_bound) { lb += (double)x; G[ms.off_a2(t) + i] += (double)pb; }
    }
    for (int i = 0; i < n3; i++) {
      T x = theta[ms.off_a3(t) + i];
      if (x > alpha_bound) { lb += (double)x; G[ms.off_a3(t) + i] += (double)pb; }
    }
  }
  for (int t = 0; t < nt; t++) {
    Sp& s = sp[t];
    int Nl = ms.tipos[t], sh = ms.shift(t), Fr = ms.Fr[t], Fa = ms.Fa[t], F = Fr + Fa;
    const T* a2 = theta + ms.off_a2(t);
    const T* a3 = theta + ms.off_a3(t);
    const T* mu = theta + ms.off_mu(t);
    const T* w = theta + ms.off_w(t);
    const T* e2 = emb + ms.emb_off(t);
    const T* e3 = e2 + nt * Fr;
    size_t n = (size_t)nf * Nl;
    std::vector<T> ndr(n * Fr), nda(n * Fa);
    for (size_t a = 0; a < n; a++) {
      for (int i = 0; i < Fr; i++) ndr[a * Fr + i] = s.nd[a * F + i];
      for (int i = 0; i < Fa; i++) nda[a * Fa + i] = s.nd[a * F + Fr + i];
    }
    std::vector<double> gn2(n * Fr, 0.0), gn3(n * Fa, 0.0), ge2(nt * Fr, 0.0);
    grad_force_radial(nf, Nl, N, nr, Fr, sh, Fbar.data(), ndr.data(), s.der2b.data(), s.im2.data(), s.rad.data(), a2,
                      e2, type_map, nt, gn2.data(), G.data() + ms.off_a2(t), ge2.data(), wpos, wbox, wb);
    grad_force_tripl(nf, Nl, N, nr, na, Fa, sh, Fbar.data(), nda.data(), s.d3s.data(), s.ang.data(), s.der3bs.data(),
                     s.der3b.data(), s.im3.data(), a3, e3, type_map, s.ntr.data(), C, gn3.data(),
                     G.data() + ms.off_a3(t), wpos, wbox, wb);
    std::vector<T> u(n * F), ebar(n), gaf(n * F);
    for (size_t a = 0; a < n; a++) {
      for (int i = 0; i < Fr; i++) u[a * F + i] = (T)gn2[a * Fr + i];
      for (int i = 0; i < Fa; i++) u[a * F + Fr + i] = (T)gn3[a * Fa + i];
      // E_b = 0.5*mean_i e_i -> dL/de_i = Ebar_b * 0.5 / N
      ebar[a] = Ebar[a / Nl] * T(0.5) / (per_atom_energy ? T(N) : T(1));
    }
    mlp_eval<T>(ms.mlp(t), (int)n, s.af.data(), mu, w, nullptr, nullptr, ebar.data(), u.data(),
                G.data() + ms.off_w(t), G.data() + ms.off_mu(t), gaf.data());
    std::vector<T> g2(n * Fr), g3(n * Fa);
    for (size_t a = 0; a < n; a++) {
      for (int i = 0; i < Fr; i++) g2[a * Fr + i] = gaf[a * F + i];
      for (int i = 0; i < Fa; i++) g3[a * Fa + i] = gaf[a * F + Fr + i];
    }
    std::vector<double> ge2b(nt * Fr, 0.0);
    grad_af_radial(nf, Nl, nr, Fr, nt, g2.data(), s.rad.data(), s.im2.data(), a2, e2, type_map,
                   G.data() + ms.off_a2(t), ge2b.data());
    grad_af_angular(nf, Nl, nr, na, Fa, g3.data(), s.ang.data(), s.d3s.data(), s.im3.data(), a3, e3, type_map,
                    s.ntr.data(), C, G.data() + ms.off_a3(t));
  }
  if (grad)
    for (int i = 0; i < P; i++) grad[i] = (T)G[i];
  if (so) {
    so->loss_e = le;
    so->loss_f = lf;
    so->loss_bound = lb;
    so->loss_v = lv;
    so->loss = (double)pe * le + (double)pb * lb + (double)pf * lf + (double)pv * lv;
  }
  return OK;
}

}  // namespace stafo

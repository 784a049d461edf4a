// C entry points of the CPU oracle (test infrastructure; see staf_oracle.hpp).
// Every function exists in a float (_f32) and a double (_f64) instantiation,
// mirroring the reference's ops_float / ops_double builds (STAF/include/staf_real.h).
#include "staf_oracle.hpp"

using namespace stafo;

template <class T>
static DescCfg<T> make_cfg(double Rc, double Rs, double Ra, int nr, int na) {
  DescCfg<T> c;
  c.Rc = (T)Rc;
  c.Rs = (T)Rs;
  c.Ra = (T)Ra;
  c.nr = nr;
  c.na = na;
  fill_repulsion(c);
  return c;
}

static ModelShape make_shape(const int* d) {
  // d = [nt, tipos[4], Fr[4], Fa[4], n_dense, width[6]]
  ModelShape m;
  m.nt = d[0];
  for (int t = 0; t < MAX_TYPES; t++) {
    m.tipos[t] = d[1 + t];
    m.Fr[t] = d[5 + t];
    m.Fa[t] = d[9 + t];
  }
  m.n_dense = d[13];
  for (int l = 0; l < MAX_DENSE; l++) m.width[l] = d[14 + l];
  return m;
}

#define STAMP(T, SFX)                                                                                                  \
  extern "C" void stafo_fill_repulsion_##SFX(double Rc, double Rs, double Ra, T* out5) {                              \
    DescCfg<T> c = make_cfg<T>(Rc, Rs, Ra, 1, 1);                                                                      \
    out5[0] = c.coeffA; out5[1] = c.coeffB; out5[2] = c.coeffC; out5[3] = c.pow_alpha; out5[4] = c.pow_beta;           \
  }                                                                                                                    \
  extern "C" int stafo_neighbour_list_##SFX(double Rc, int nr, int N, const T* pos, const T* box, T* frac, int* with,  \
                                            int* howmany, T* d2, int* ncell3) {                                        \
    return neighbour_list<T>((T)Rc, nr, N, pos, box, frac, with, howmany, d2, ncell3);                                 \
  }                                                                                                                    \
  extern "C" int stafo_descriptors_##SFX(double Rc, double Rs, double Ra, int nr, int na, int nf, int N, const T* pos, \
                                         const T* box, T* raddescr, T* angdescr, T* des3bsupp, int* intmap2b,          \
                                         int* intmap3b, T* der2b, T* der3b, T* der3bsupp, int* numtriplet,             \
                                         T* nbr_d2) {                                                                  \
    DescCfg<T> c = make_cfg<T>(Rc, Rs, Ra, nr, na);                                                                    \
    return descriptors<T>(c, nf, N, pos, box, raddescr, angdescr, des3bsupp, intmap2b, intmap3b, der2b, der3b,         \
                          der3bsupp, numtriplet, nbr_d2);                                                              \
  }                                                                                                                    \
  extern "C" void stafo_af_radial_##SFX(int nf, int Nl, int nr, int Fr, const T* raddescr, const int* intmap2b,        \
                                        const T* alpha2b, const T* e2, const int* type_map, T* out) {                  \
    af_radial<T>(nf, Nl, nr, Fr, raddescr, intmap2b, alpha2b, e2, type_map, out);                                      \
  }                                                                                                                    \
  extern "C" void stafo_af_angular_##SFX(int nf, int Nl, int nr, int na, int Fa, const T* angdescr, const T* ds,       \
                                         const int* intmap3b, const T* alpha3b, const T* e3, const int* type_map,      \
                                         const int* numtriplet, T* out) {                                              \
    af_angular<T>(nf, Nl, nr, na, Fa, angdescr, ds, intmap3b, alpha3b, e3, type_map, numtriplet, out);                 \
  }                                                                                                                    \
  extern "C" void stafo_force_radial_##SFX(int nf, int Nl, int N, int nr, int Fr, int shift, const T* netderiv,        \
                                           const T* der2b, const int* intmap2b, const T* raddescr, const T* alpha2b,   \
                                           const T* e2, const int* type_map, T* force, const T* pos,            \
                                           const T* box, T* virial) {                                                   \
    std::vector<double> F((size_t)nf * 3 * N, 0.0), W((size_t)nf * 9, 0.0);                                            \
    force_radial<T>(nf, Nl, N, nr, Fr, shift, netderiv, der2b, intmap2b, raddescr, alpha2b, e2, type_map, F.data(),    \
                    pos, box, virial ? W.data() : nullptr);                                                            \
    for (size_t i = 0; i < F.size(); i++) force[i] = (T)F[i];                                                          \
    if (virial) for (size_t i = 0; i < W.size(); i++) virial[i] = (T)W[i];                                             \
  }                                                                                                                    \
  extern "C" void stafo_force_tripl_##SFX(int nf, int Nl, int N, int nr, int na, int Fa, int shift, const T* netderiv, \
                                          const T* ds, const T* angdescr, const T* der3bsupp, const T* der3b,          \
                                          const int* intmap3b, const T* alpha3b, const T* e3, const int* type_map,     \
                                          const int* numtriplet, T* force, const T* pos, const T* box,                 \
                                          T* virial) {                                                                 \
    std::vector<double> F((size_t)nf * 3 * N, 0.0), W((size_t)nf * 9, 0.0);                                            \
    force_tripl<T>(nf, Nl, N, nr, na, Fa, shift, netderiv, ds, angdescr, der3bsupp, der3b, intmap3b, alpha3b, e3,      \
                   type_map, numtriplet, F.data(), pos, box, virial ? W.data() : nullptr);                             \
    for (size_t i = 0; i < F.size(); i++) force[i] = (T)F[i];                                                          \
    if (virial) for (size_t i = 0; i < W.size(); i++) virial[i] = (T)W[i];                                             \
  }                                                                                                                    \
  extern "C" void stafo_grad_af_radial_##SFX(int nf, int Nl, int nr, int Fr, int nt, const T* prevgrad,                \
                                             const T* raddescr, const int* intmap2b, const T* alpha2b, const T* e2,    \
                                             const int* type_map, T* g_alpha, T* g_emb) {                              \
    std::vector<double> ga(nt * Fr, 0.0), ge(nt * Fr, 0.0);                                                            \
    grad_af_radial<T>(nf, Nl, nr, Fr, nt, prevgrad, raddescr, intmap2b, alpha2b, e2, type_map, ga.data(), ge.data());  \
    for (int i = 0; i < nt * Fr; i++) { g_alpha[i] = (T)ga[i]; g_emb[i] = (T)ge[i]; }                                  \
  }                                                                                                                    \
  extern "C" void stafo_grad_af_angular_##SFX(int nf, int Nl, int nr, int na, int Fa, int C, const T* prevgrad,        \
                                              const T* angdescr, const T* ds, const int* intmap3b, const T* alpha3b,   \
                                              const T* e3, const int* type_map, const int* numtriplet, T* g_alpha3,    \
                                              T* g_emb3) {                                                             \
    std::vector<double> ga((size_t)C * 3 * Fa, 0.0);                                                                   \
    grad_af_angular<T>(nf, Nl, nr, na, Fa, prevgrad, angdescr, ds, intmap3b, alpha3b, e3, type_map, numtriplet, C,     \
                       ga.data());                                                                                     \
    for (int i = 0; i < C * 3 * Fa; i++) g_alpha3[i] = (T)ga[i];                                                       \
    for (int i = 0; i < C * Fa; i++) g_emb3[i] = T(0);                                                                 \
  }                                                                                                                    \
  extern "C" void stafo_grad_force_radial_##SFX(int nf, int Nl, int N, int nr, int Fr, int nt, int shift,              \
                                                const T* prevgrad, const T* netderiv, const T* der2b,                  \
                                                const int* intmap2b, const T* raddescr, const T* alpha2b,              \
                                                const T* e2, const int* type_map, T* gradnet, T* g_alpha, T* g_emb,    \
                                                const T* pos, const T* box, const T* wbar) {                           \
    std::vector<double> gn((size_t)nf * Nl * Fr, 0.0), ga(nt * Fr, 0.0), ge(nt * Fr, 0.0);                             \
    grad_force_radial<T>(nf, Nl, N, nr, Fr, shift, prevgrad, netderiv, der2b, intmap2b, raddescr, alpha2b, e2,         \
                         type_map, nt, gn.data(), ga.data(), ge.data(), pos, box, wbar);                               \
    for (size_t i = 0; i < gn.size(); i++) gradnet[i] = (T)gn[i];                                                      \
    for (int i = 0; i < nt * Fr; i++) { g_alpha[i] = (T)ga[i]; g_emb[i] = (T)ge[i]; }                                  \
  }                                                                                                                    \
  extern "C" void stafo_grad_force_tripl_##SFX(int nf, int Nl, int N, int nr, int na, int Fa, int C, int shift,        \
                                               const T* prevgrad, const T* netderiv, const T* ds, const T* angdescr,   \
                                               const T* der3bsupp, const T* der3b, const int* intmap3b,                \
                                               const T* alpha3b, const T* e3, const int* type_map,                     \
                                               const int* numtriplet, T* gradnet, T* g_alpha3, T* g_ck, const T* pos,  \
                                               const T* box, const T* wbar) {                                          \
    std::vector<double> gn((size_t)nf * Nl * Fa, 0.0), ga((size_t)C * 3 * Fa, 0.0);                                    \
    grad_force_tripl<T>(nf, Nl, N, nr, na, Fa, shift, prevgrad, netderiv, ds, angdescr, der3bsupp, der3b, intmap3b,    \
                        alpha3b, e3, type_map, numtriplet, C, gn.data(), ga.data(), pos, box, wbar);                   \
    for (size_t i = 0; i < gn.size(); i++) gradnet[i] = (T)gn[i];                                                      \
    for (int i = 0; i < C * 3 * Fa; i++) g_alpha3[i] = (T)ga[i];                                                       \
    for (int i = 0; i < C * Fa; i++) g_ck[i] = T(0);                                                                   \
  }                                                                                                                    \
  extern "C" void stafo_mlp_eval_##SFX(int n_in, int n_dense, const int* width, int n_atoms, const T* af,              \
                                       const T* mu, const T* w, T* e_out, T* netderiv_out, const T* ebar, const T* u,  \
                                       T* g_w, T* g_mu, T* g_af) {                                                     \
    MlpShape sh;                                                                                                       \
    sh.n_in = n_in;                                                                                                    \
    sh.n_dense = n_dense;                                                                                              \
    for (int l = 0; l < n_dense; l++) sh.width[l] = width[l];                                                          \
    if (g_w) {                                                                                                         \
      std::vector<double> gw(sh.n_weights(), 0.0), gm(n_in, 0.0);                                                      \
      mlp_eval<T>(sh, n_atoms, af, mu, w, e_out, netderiv_out, ebar, u, gw.data(), gm.data(), g_af);                   \
      for (int i = 0; i < sh.n_weights(); i++) g_w[i] = (T)gw[i];                                                      \
      for (int i = 0; i < n_in; i++) g_mu[i] = (T)gm[i];                                                               \
    } else {                                                                                                           \
      mlp_eval<T>(sh, n_atoms, af, mu, w, e_out, netderiv_out, nullptr, nullptr, nullptr, nullptr, nullptr);           \
    }                                                                                                                  \
  }                                                                                                                    \
  extern "C" int stafo_energy_force_grad_##SFX(double Rc, double Rs, double Ra, int nr, int na, const int* shape_desc, \
                                               int nf, const T* pos, const T* box, const int* type_map,                \
                                               const T* theta, const T* emb, int per_atom_energy, T* energy,           \
                                               T* force, int with_grad, const T* e_label, const T* f_label, double pe, \
                                               double pf, double pb, double alpha_bound, int loss_kind,                \
                                               double* losses4, T* grad) {                                             \
    DescCfg<T> c = make_cfg<T>(Rc, Rs, Ra, nr, na);                                                                    \
    ModelShape ms = make_shape(shape_desc);                                                                            \
    StepOut so = {0, 0, 0, 0, 0};                                                                                      \
    int st = energy_force_grad<T>(c, ms, nf, pos, box, type_map, theta, emb, per_atom_energy != 0, energy, force,      \
                                  with_grad != 0, e_label, f_label, (T)pe, (T)pf, (T)pb, (T)alpha_bound, loss_kind,    \
                                  &so, grad);                                                                          \
    if (losses4) { losses4[0] = so.loss; losses4[1] = so.loss_e; losses4[2] = so.loss_bound; losses4[3] = so.loss_f; } \
    return st;                                                                                                         \
  }                                                                                                                    \
  /* the same with the virial term of full_train_e_f_v: losses5 = loss, loss_e, loss_bound, loss_f, loss_v */         \
  extern "C" int stafo_energy_force_virial_grad_##SFX(                                                                 \
      double Rc, double Rs, double Ra, int nr, int na, const int* shape_desc, int nf, const T* pos, const T* box,      \
      const int* type_map, const T* theta, const T* emb, int per_atom_energy, T* energy, T* force, T* virial,          \
      int with_grad, const T* e_label, const T* f_label, const T* v_label, double pe, double pf, double pv, double pb, \
      double alpha_bound, int loss_kind, double* losses5, T* grad) {                                                   \
    DescCfg<T> c = make_cfg<T>(Rc, Rs, Ra, nr, na);                                                                    \
    ModelShape ms = make_shape(shape_desc);                                                                            \
    StepOut so = {0, 0, 0, 0, 0};                                                                                      \
    int st = energy_force_grad<T>(c, ms, nf, pos, box, type_map, theta, emb, per_atom_energy != 0, energy, force,      \
                                  with_grad != 0, e_label, f_label, (T)pe, (T)pf, (T)pb, (T)alpha_bound, loss_kind,    \
                                  &so, grad, with_grad ? v_label : (const T*)nullptr, (T)pv, virial);                  \
    if (losses5) {                                                                                                     \
      losses5[0] = so.loss; losses5[1] = so.loss_e; losses5[2] = so.loss_bound; losses5[3] = so.loss_f;                \
      losses5[4] = so.loss_v;                                                                                          \
    }                                                                                                                  \
    return st;                                                                                                         \
  }

STAMP(float, f32)
STAMP(double, f64)

extern "C" int stafo_n_params(const int* shape_desc) { return make_shape(shape_desc).n_params(); }
extern "C" int stafo_n_emb(const int* shape_desc) { return make_shape(shape_desc).n_emb(); }
extern "C" void stafo_offsets(const int* shape_desc, int t, int* out6) {
  ModelShape m = make_shape(shape_desc);
  out6[0] = m.off_a2(t);
  out6[1] = m.off_a3(t);
  out6[2] = m.off_mu(t);
  out6[3] = m.off_w(t);
  out6[4] = m.emb_off(t);
  out6[5] = m.block_size(t);
}
extern "C" int stafo_max_threads() {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
extern "C" void stafo_set_threads(int n) {
#ifdef _OPENMP
  omp_set_num_threads(n);
#else
  (void)n;
#endif
}

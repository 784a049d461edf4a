// Driver around the reference's own CPU neighbour list (test infrastructure).
// It calls getList / updateList / calculateInteractionMapWithCutoffDistanceOrdered
// of STAF/src/descriptor_builder/cell_list.cu.cc (lines 40, 143, 1080), which are
// compiled from the reference tree where it lies; no reference source is copied.
// `real` is fixed at compile time (-DSTAF_REAL_DOUBLE), so this file is built
// twice: libref_nl_f32.so and libref_nl_f64.so.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include "vector.h"
#include "interaction_map.h"
#include "cell_list.h"

extern "C" int ref_real_bytes() { return (int)sizeof(real); }

// pos: Cartesian [N,3]; box: [Lx,xy,xz,Ly,yz,Lz].  Fractional coordinates are
// formed exactly as descriptor_builder/reforce.cc:283-299 + celle_gpu.cu.cc:11-28.
extern "C" int ref_neighbour_list(double Rc, int nr, int N, const real* pos, const real* box, int* with,
                                  int* howmany, real* d2, int* ncell3) {
  real I[6];
  I[0] = real(1.) / box[0];
  I[1] = -box[1] / (box[0] * box[3]);
  I[2] = (box[1] * box[4]) / (box[0] * box[3] * box[5]) - box[2] / (box[0] * box[5]);
  I[3] = real(1.) / box[3];
  I[4] = -box[4] / (box[3] * box[5]);
  I[5] = real(1.) / box[5];
  vector* fr = (vector*)calloc(N, sizeof(vector));
  for (int p = 0; p < N; p++) {
    real px = pos[3 * p], py = pos[3 * p + 1], pz = pos[3 * p + 2];
    fr[p].x = (I[0] * px + I[1] * py + I[2] * pz);
    fr[p].y = (I[3] * py + I[4] * pz);
    fr[p].z = (I[5] * pz);
  }
  listcell* l = getList(box, (real)Rc, N);
  ncell3[0] = l->NumberCells_x;
  ncell3[1] = l->NumberCells_y;
  ncell3[2] = l->NumberCells_z;
  updateList(l, fr, N);
  // generous row width: the reference row has no bound check while inserting
  int width = 4 * nr + 64;
  interactionmap* ime = createInteractionMap(N, width);
  resetInteractionMap(ime);
  calculateInteractionMapWithCutoffDistanceOrdered(l, ime, fr, box, (real)Rc);
  int over = 0;
  for (int i = 0; i < N; i++) {
    howmany[i] = ime->howmany[i];
    if (ime->howmany[i] > nr) over = 1;
    int n = ime->howmany[i] < nr ? ime->howmany[i] : nr;
    for (int k = 0; k < n; k++) {
      with[i * nr + k] = ime->with[i][k];
      d2[i * nr + k] = ime->rij2[i][k];
    }
  }
  freeInteractionMap(ime);
  freeList(l);
  free(fr);
  return over;
}

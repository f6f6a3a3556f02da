// The launch switch of a kernel family: every family (a shared object of its own) links this file and so has its own
// copy, which ccb_set_pdl of that family sets.
#include "common.cuh"

int g_ccb_pdl = 0;

// 1: the products of the library may overlap the end of their predecessor; 2: every kernel (see common.cuh)
CCB_API int ccb_set_pdl(int on) {
  g_ccb_pdl = on < 0 ? 0 : (on > 2 ? 2 : on);
  return 0;
}

// N-dimensional device mesh coordinate math (row-major over ranks) and sub-group enumeration.
// Same semantics as the reference DeviceMesh (process_group/device_mesh.cpp:64-121,143-177): the
// process group of axis `a` that contains `rank` is the set of ranks that share every other
// coordinate, ordered by their coordinate on `a`; grouping is by rank index only, so correctness never
// depends on placement.  Communicator creation itself is done by the caller (torch.distributed).
#include <stdint.h>

#include "../kernels/host_utils.h"

using namespace cpb;

extern "C" int cpb_mesh_coords(const int* shape, int ndim, int rank, int* coords_out) {
  long total = 1;
  for (int i = 0; i < ndim; ++i) { if (shape[i] <= 0) return set_error(CPB_ERR_ARG, "mesh: non-positive extent"); total *= shape[i]; }
  if (rank < 0 || rank >= total) return set_error(CPB_ERR_ARG, "mesh: rank %d outside mesh of %ld", rank, total);
  for (int i = ndim - 1; i >= 0; --i) { coords_out[i] = rank % shape[i]; rank /= shape[i]; }
  return CPB_OK;
}

extern "C" int cpb_mesh_rank(const int* shape, int ndim, const int* coords) {
  int r = 0;
  for (int i = 0; i < ndim; ++i) {
    if (coords[i] < 0 || coords[i] >= shape[i]) return -1;
    r = r * shape[i] + coords[i];
  }
  return r;
}

// ranks_out[shape[axis]]: members of the axis group containing `rank`, in axis-coordinate order.
extern "C" int cpb_mesh_group_ranks(const int* shape, int ndim, int rank, int axis, int* ranks_out) {
  if (axis < 0 || axis >= ndim) return set_error(CPB_ERR_ARG, "mesh: axis %d out of range", axis);
  int coords[16];
  if (ndim > 16) return set_error(CPB_ERR_ARG, "mesh: too many dimensions");
  int rc = cpb_mesh_coords(shape, ndim, rank, coords);
  if (rc) return rc;
  for (int c = 0; c < shape[axis]; ++c) {
    coords[axis] = c;
    ranks_out[c] = cpb_mesh_rank(shape, ndim, coords);
  }
  return CPB_OK;
}

// Group "colour": identical for exactly the ranks that share an axis group.
extern "C" int cpb_mesh_group_color(const int* shape, int ndim, int rank, int axis) {
  int coords[16];
  if (ndim > 16 || cpb_mesh_coords(shape, ndim, rank, coords)) return -1;
  int color = 0;
  for (int i = 0; i < ndim; ++i) if (i != axis) color = color * shape[i] + coords[i];
  return color;
}

// Work units of the Gram norm pass: which 128 x 128 blocks of a sample's T x T plane one tile covers.
// Plain inline functions for host and device (no CUDA types), so the enumeration can be checked on a CPU.
#pragma once
#ifndef __CUDACC__
#ifndef __host__
#define __host__
#endif
#ifndef __device__
#define __device__
#endif
#endif

namespace fdp {

// ---- Gram work units -----------------------------------------------------------------------------------
// Row i of the upper block triangle holds blocks (i, i..nb-1).  Rows with an odd block count (every
// second row) are paired (a, a+2): block (a, a+2) is computed as its mirror image (a+2, a) in row a+2
// instead -- the summand (G G^T)(X X^T) is symmetric -- so both rows end up with an even count and
// every unit is a pair of blocks of one row.  Only when the number of odd rows is odd does one row keep
// a single-block unit.  Unit u of a sample -> t-block i and s-blocks j1, j2 (j2 = -1: single block).
__host__ __device__ inline int gram_row_len(int nb, int i, int& role) {
  const int p = (nb - 1) & 1;      // odd rows are i = p, p+2, ...
  int len = nb - i;
  role = 0;                        // 0: untouched row, 1: gives block (i, i+2) away, 2: receives (i, i-2)
  if (i >= p && ((i - p) & 1) == 0) {
    const int m = (i - p) >> 1;
    if (m & 1) { role = 2; len += 1; }
    else if (i + 2 < nb) { role = 1; len -= 1; }
  }
  return len;
}
__host__ __device__ inline int gram_col(int i, int role, int e) {
  if (role == 2) return e == 0 ? i - 2 : i + e - 1;
  if (role == 1) return e >= 2 ? i + e + 1 : i + e;
  return i + e;
}
__host__ __device__ inline int gram_units(int nb) {
  int n = 0, role;
  for (int i = 0; i < nb; ++i) n += (gram_row_len(nb, i, role) + 1) >> 1;
  return n;
}
__host__ __device__ inline void gram_decode(int nb, int u, int& i, int& j1, int& j2) {
  int role;
  for (i = 0; i < nb; ++i) {
    const int len = gram_row_len(nb, i, role);
    const int n = (len + 1) >> 1;
    if (u < n) {
      j1 = gram_col(i, role, 2 * u);
      j2 = (2 * u + 1 < len) ? gram_col(i, role, 2 * u + 1) : -1;
      return;
    }
    u -= n;
  }
  i = j1 = 0; j2 = -1;   // not reached for u < gram_units(nb)
}

}  // namespace fdp

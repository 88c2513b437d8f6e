// Launch-shape selection shared by the row-wise kernels.
//
// A row is processed by a GROUP of G threads; every thread keeps VPT 128-bit
// vectors of the row in registers, so a group covers G*VPT vectors. A block
// holds threads/G groups that work on different rows at the same time. Rows
// whose byte width is not a multiple of 16, or that do not fit G*VPT for any
// listed shape, take the generic multi-pass kernels instead.
#pragma once

#include <cstdio>

#include "evg_common.cuh"

namespace evg {

// (G, VPT) shapes that are instantiated. Keep in sync with pick_rowcfg().
#define EVG_ROWCFG_LIST(X) \
  X(32, 1) X(32, 2) X(32, 4) X(64, 3) X(64, 4) X(64, 8) X(128, 3) X(128, 4) X(256, 2) X(256, 3) \
  X(256, 4) X(512, 1) X(512, 4) X(1024, 4) X(1024, 8)

// Upper bound on the block size a (G, VPT) kernel may be launched with; it is
// also the kernel's __launch_bounds__, which fixes the register budget.
constexpr int rowcfg_max_threads(int G) { return G > 512 ? 1024 : 512; }

struct RowCfg {
  int G = 0;
  int VPT = 0;
  int threads = 0;  // block size, a multiple of G
};

inline bool rowcfg_listed(int G, int VPT) {
#define EVG_X(g, v) if (G == g && VPT == v) return true;
  EVG_ROWCFG_LIST(EVG_X)
#undef EVG_X
  return false;
}

// Returns false when no register-resident shape fits (use the generic kernel).
// `op` prefixes the tuning keys ("<op>.group", "<op>.vpt", "<op>.threads").
// `prefer_threads` is the default block size (0: one group of >= 256 threads);
// `narrow` prefers (256, 2) over (128, 4) for 512-vector rows, which halves the
// per-thread accumulator count of kernels that keep two column sums.
inline bool pick_rowcfg(const char* op, int64_t nvec, RowCfg& cfg, int prefer_threads = 0,
                        bool narrow = false) {
  if (nvec <= 0 || nvec > 8192) return false;
  char key[96];
  snprintf(key, sizeof(key), "%s.group", op);
  int fg = tune(key);
  snprintf(key, sizeof(key), "%s.vpt", op);
  int fv = tune(key);
  snprintf(key, sizeof(key), "%s.threads", op);
  int ft = tune(key);
  int G, V;
  if (fg > 0 && fv > 0 && rowcfg_listed(fg, fv) && (int64_t)fg * fv >= nvec) {
    G = fg; V = fv;
  } else if (nvec <= 32) { G = 32; V = 1; }
  else if (nvec <= 64) { G = 32; V = 2; }
  else if (nvec <= 128) { G = 32; V = 4; }
  else if (nvec <= 192) { G = 64; V = 3; }  // e.g. 1536 bf16 columns: no idle quarter of a group
  else if (nvec <= 256) { G = 64; V = 4; }
  else if (nvec <= 384) { G = 128; V = 3; }  // e.g. 3072 bf16 columns
  else if (nvec <= 512 && narrow) { G = 256; V = 2; }
  else if (nvec <= 512) { G = 128; V = 4; }
  else if (nvec <= 768) { G = 256; V = 3; }  // e.g. 5120 bf16 columns: no idle quarter of a group
  else if (nvec <= 1024) { G = 256; V = 4; }
  else if (nvec <= 2048) { G = 512; V = 4; }
  else if (nvec <= 4096) { G = 1024; V = 4; }
  else { G = 1024; V = 8; }
  int threads = G >= 256 ? G : 256;
  if (prefer_threads > 0 && prefer_threads % G == 0 && prefer_threads <= rowcfg_max_threads(G) &&
      (G == 32 || prefer_threads / G <= 15))
    threads = prefer_threads;
  if (ft > 0 && ft % G == 0 && ft <= rowcfg_max_threads(G) && (G == 32 || ft / G <= 15))
    threads = ft;
  cfg.G = G; cfg.VPT = V; cfg.threads = threads;
  return true;
}

// Number of persistent blocks: enough to fill every SM at the kernel's
// occupancy, never more than there are row slots.
template <typename Kernel>
inline int persistent_grid(Kernel kernel, int threads, size_t smem, int64_t rows, int groups,
                           int max_blocks = 1 << 30) {
  int occ = 0;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, threads, smem);
  if (occ < 1) occ = 1;
  int64_t want = (int64_t)device_info().sm_count * occ;
  int64_t need = (rows + groups - 1) / groups;
  if (want > need) want = need;
  if (want > max_blocks) want = max_blocks;
  if (want < 1) want = 1;
  return (int)want;
}

}  // namespace evg

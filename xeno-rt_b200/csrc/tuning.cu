// Choices among kernel variants that a caller may force, for comparison and for tests.  They are
// arguments, not environment: the Python side sets them through xrt_set_tuning (csrc/ops.py,
// `Tuning`), nothing in this library reads the environment.
#include "common.cuh"

namespace xrt {

static Tuning g_tuning;

const Tuning& tuning() { return g_tuning; }

}  // namespace xrt

// key: 0 pdl (1 on, 0 off); 1 decode_attention (0 auto, 1 heads as rows, 2 cp.async copies, 3 no
// clusters); 2 gemm_tile_rows (0 auto, 128, 256); 3 decode_gemm_clusters (1 on, 0 off); 4 decode_cluster_pairs
// (decode attention merges its splits as clusters up to so many (token, kv head) pairs).
XRT_EXPORT int xrt_set_tuning(int key, int value) {
  using xrt::g_tuning;
  switch (key) {
    case 0: g_tuning.pdl = value != 0; return XRT_OK;
    case 1: if (value < 0 || value > 3) return XRT_ERR_ARGUMENT; g_tuning.decode_attention = value; return XRT_OK;
    case 2: if (value != 0 && value != 128 && value != 256) return XRT_ERR_ARGUMENT; g_tuning.gemm_tile_rows = value; return XRT_OK;
    case 3: g_tuning.decode_gemm_clusters = value != 0; return XRT_OK;
    case 4: if (value < 0) return XRT_ERR_ARGUMENT; g_tuning.decode_cluster_pairs = value; return XRT_OK;
    default: return XRT_ERR_ARGUMENT;
  }
}

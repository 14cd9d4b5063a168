// Device-side parameter block of the attention forward kernels and the enums
// that select a kernel instantiation.  Filled by the host layer from the public
// C struct after validation; never seen by callers of the library.
#pragma once
#include <stdint.h>

namespace flb {

enum ScoreMod : int {
  SCORE_NONE = 0,
  SCORE_ALIBI = 1,
  SCORE_SOFTCAP = 2,
  SCORE_BIAS = 3,
  // kernel-internal modes (never in the public struct): the back-to-back product
  // O = f(Q K^T * scale) V without softmax, K given as [S][E] rows or as [E][S] (keys contiguous)
  SCORE_B2B = 4,
  SCORE_B2BT = 5,
  // additive biases with the pair bias (shared by every row of a batch element) resident in shared
  // memory: a CTA keeps one (head, query tile) and walks a range of rows
  SCORE_BIAS_RES = 6
};
// pointwise function between the two products of the back-to-back mode
enum Pointwise : int { PW_IDENTITY = 0, PW_RELU = 1, PW_TANH = 2, PW_SIGMOID = 3 };
enum MaskKind : int {
  MASK_NONE = 0,
  MASK_CAUSAL = 1,    // keep j <= i
  MASK_SLIDING = 2,   // keep i - window <= j <= i
  MASK_PREFIX = 3,    // keep j <= max(prefix_len[n] - 1, i)
  MASK_DOCUMENT = 4   // keep doc[n][i] == doc[n][j] (and j <= i when causal)
};

// Tile classes written by the block-map builder (one byte per (n, q-tile, kv-tile)).
enum TileClass : uint8_t { TILE_SKIP = 0, TILE_PARTIAL = 1, TILE_FULL = 2 };

constexpr int kTileM = 128;  // query rows per softmax warpgroup (one TMEM lane each)
constexpr int kTileN = 128;  // keys per step

struct KernelParams {
  // problem: n in [0,N), h in [0,H) output heads, q rows L, keys S
  int N, H, L, S;
  int G;            // query heads per kv head (kv head = h / G)
  int diff_heads;   // differential attention: second branch reads q/k head h + diff_heads
  int evo_inner;    // batch index n = b * evo_inner + r (bias broadcasting); 1 otherwise
  // output [n][h][l][EV], EV contiguous, element strides
  void* o;
  int64_t o_sn, o_sh, o_sl;
  float* lse;       // optional [n][h][l] fp32 log-sum-exp (natural log), or null
  int64_t lse_sn, lse_sh;
  // scores
  float scale;        // applied to q.k
  float scale_log2;   // scale * log2(e)
  float alibi_log2_slope_step;  // -8 / n_heads: slope_h = 2^((alibi_head0 + h + 1) * step)
  int alibi_head0;
  float softcap;      // cap
  int pointwise;      // Pointwise, back-to-back mode only
  // additive biases (bf16), row pointer = base + b*sb + r*sr + h*sh + i*sl, keys contiguous
  const void* bias[2];
  int64_t bias_sb[2], bias_sr[2], bias_sh[2], bias_sl[2];
  int bias_vec[2];  // rows are 16-byte aligned: 128-bit loads allowed
  // resident-bias kernel: bias[0] is the per-row key vector (or null; strides sb, sr, sh), the pair
  // bias comes through a tensor map with coordinates (key, query, head * pair_h, batch * pair_b);
  // every CTA walks res_rows rows of one batch element, res_chunks CTAs cover its evo_inner rows
  int pair_h, pair_b;
  int res_rows, res_chunks;
  int res_slots;  // slots (one tile each) of each stage's K/V ring; the bias tiles lie behind the rings
  // resident-bias kernel with the key vector added by the tensor cores: per (row, key) a 16-column
  // bf16 row [hi, lo, 0 ...] of bias / scale, written by keyvec_rows_kernel in the shared-memory image
  // of a 32-byte swizzled tile (4 KB per 128 keys); nullptr: the softmax threads add the vector
  const uint8_t* keyvec_rows;
  int keyvec_tiles;  // key tiles per row (row stride = keyvec_tiles * 4096 bytes)
  // masks
  int causal;                // document mask: also require j <= i
  int window;                // sliding window (keys i-window .. i)
  const int32_t* prefix_len; // per n, or null -> prefix_scalar
  int prefix_scalar;
  const int64_t* doc;        // [N][L] document ids
  int64_t doc_sn;
  const int32_t* map_range;  // [N][nq][2] first / one-past-last kv tile to visit
  const uint8_t* map_cls;    // [N][nq][nkv] TileClass
  const int32_t* map_sorted; // [N] 1 when the sequence's ids never decrease
  const int32_t* map_runs;   // [N][L][2] first / last index of the run of equal ids around i
  // differential attention epilogue
  float lambda;
  int rms_norm;
  float rms_eps;
  // fp16 P.V of differential attention: bits of max |v| over the whole V tensor, found by v_absmax_kernel;
  // V is multiplied by the power of two that brings that maximum to [2^13, 2^14) on its way to fp16
  // (the RMS normalisation makes the result independent of it, eps scaled alike)
  const uint32_t* v_absmax;
  float inv_ev;     // 1 / (true value width): the mean of the RMS normalisation
  int v_halves;     // 2: value heads wider than the kernel; CTA pairs take one half of the columns each
  int v_exchange;   // the two CTAs of a pair run as a cluster and swap their rows' sums of squares
  // bookkeeping
  int nq_blocks;   // CTAs along the query axis
  int sec_bh;      // (batch, head) pairs per L2 section: their K/V together fit in L2
  int* status;     // device int32, 0 = ok; may be null
  int* status_host;  // pinned host int32 (device-accessible) that receives a copy; may be null
  uint32_t wait_limit_us;  // limit of every device-side wait
  int withhold_loads;      // wait self-test: the producer issues no loads
};

// status word layout: (code << 24) | (barrier id << 16) | (block index & 0xffff)
constexpr int kStatusTimeout = 1;

}  // namespace flb

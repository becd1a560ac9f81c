// Internal interfaces between the host layer (capi.cc, planner.cc) and the kernels.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <string>

#include "qfg.h"

namespace qfg {

constexpr int kMaxSeg = QFG_MAX_WEIGHTS;
constexpr int kMaxOut = QFG_MAX_OUTPUTS;
constexpr int kMaxRows = 8;  // rows of x one launch handles (the n = 8 side of m16n8k16)
#ifndef QFG_MAX_WARPS
#define QFG_MAX_WARPS 20
#endif
constexpr int kMaxWarps = QFG_MAX_WARPS;  // warps per CTA of the warp-ring kernel (sets its register budget)

enum WeightMode : int { kBf16 = 0, kFp8 = 1, kNvfp4 = 2 };

// Per-mode geometry of the streaming kernel: a thread owns `kColsPerThread` columns of four
// weight rows per k-step, fetched as one shared-memory load of `kBytesPerThread` per row.
struct ModeGeom {
  int cols_per_thread;   // 8 (BF16), 16 (FP8), 16 (NVFP4)
  int bytes_per_thread;  // 16, 16, 8
  int cols_per_warp;     // 8 thread groups side by side
  int bytes_per_warp;    // per weight row
};
// `wide` = 2: the NVFP4 direct kernel's variant whose warps cover 256 columns (a thread owns two
// 16-column groups 128 columns apart).
inline ModeGeom GeomOf(int mode, int wide = 1) {
  switch (mode) {
    case kBf16: return {8, 16, 64, 128};
    case kFp8: return {16, 16, 128, 128};
    default: return wide == 2 ? ModeGeom{16, 8, 256, 128} : ModeGeom{16, 8, 128, 64};
  }
}
// The NVFP4 warp rings copy their scale bytes through L1, where the four column warps that share a 32-byte sector of
// scales fetch it from L2 once.  That needs L1 room beside the CTA's shared memory: measured on the 151936-column
// head, 102.6 us with a 132 KB carve-out, 108 us with 196 KB, 153 us with 228 KB (the lines are evicted before they
// are shared).  The ring depth is chosen to stay within the 164 KB carve-out where a depth fits it (kL1FriendlySmem:
// that carve-out less the kernels' static shared memory), and past the 196 KB carve-out (kL1UsableSmem) the scale
// bytes bypass L1 like everything else.
constexpr size_t kL1FriendlySmem = 161 * 1024;
constexpr size_t kL1UsableSmem = 193 * 1024;
// Bytes of one k-step of one warp in the ring of the direct kernel.
inline int RingSlotBytes(int mode) { return mode == kNvfp4 ? 1584 : 2048; }
// The same for the tcgen05 kernel, which keeps the older slot layout.
inline int DirectSlotBytes(int mode, int wide) {
  if (mode != kNvfp4) return 4 * 32 * 16;
  const int w = wide == 2 ? 2 : 1;
  return 16 * (64 * w + 16) + 32 + 16 * 32 + 96;
}

// Launch geometry.  It depends on (K, segment widths, weight type) only - never on the
// number of rows - so that a row's reduction order is the same in every call.
struct Plan {
  int wn = 4;       // warps side by side along N
  int wk = 2;       // warps splitting each stage along K
  int ks = 1;       // k-steps (16 rows) per warp per stage
  int stages = 4;   // depth of the shared-memory ring
  int cluster = 1;  // CTAs splitting K, reduced through distributed shared memory
  int tiles[kMaxSeg] = {0, 0, 0, 0};  // column tiles per segment
  int gran = 16;    // columns per granule of the balanced column partition
  int direct = 1;   // 1: warp-private cp.async rings, no CTA barrier in the K loop; 2: warps stream straight into
                    // registers (BF16 / FP8); 0: CTA-wide ring
  int wide = 1;     // NVFP4 direct kernel: 16-column groups per thread (1 or 2)
  int tail = 0;     // fused LM head: trailing 128-column groups whose K range is split over all CTAs (see GemmParams)
  int tc = 0;       // NVFP4: 1 = tcgen05 kernel (wn x wk warps feed tensor memory, one warp issues the MMAs, wk more
                    // warps run mma.sync on up to 128 columns past wn x 128)
  int warps() const { return tc ? wn * wk + 1 + wk : wn * wk; }
  int threads() const { return 32 * warps(); }
  int rows_per_stage() const { return 16 * wk * ks; }
};

// Columns a CTA of this plan can hold.
inline int PlanMaxCols(const Plan& plan, int mode) {
  const ModeGeom g = GeomOf(mode, plan.direct ? plan.wide : 1);
  return (plan.wn + (plan.tc ? 1 : 0)) * g.cols_per_warp;
}

struct Segment {
  const uint8_t* w = nullptr;
  const float* w_scale = nullptr;
  long long pitch = 0;        // bytes per stored row
  long long total_bytes = 0;  // K * pitch
  int n = 0;
  int tile_begin = 0;
  int tiles = 0;
  int granules = 0;
  int gran_quot = 0;  // granules / tiles and granules % tiles: tile t starts at granule t * quot + t * rem / tiles
  int gran_rem = 0;   // (32-bit arithmetic on the device; tiles < 65536)
  int out_begin = 0;
  int out_end = 0;
  int tail_cols = 0;  // trailing columns left out of the column tiles (fused LM head, see GemmParams::tail_groups)
  int vec = 16;   // cp.async width for the weight bytes of a row
  int svec = 4;   // cp.async width for the NVFP4 scale bytes of a row
};

constexpr int kExchangeSpin = 1 << 22;  // default bound of the wait for a peer's words (iterations of about 50 ns)

struct GemmParams {
  const uint16_t* x = nullptr;  // BF16 [M, K]
  int M = 0;
  int K = 0;
  int nseg = 0;
  Segment seg[kMaxSeg];
  uint16_t* out[kMaxOut] = {};
  int col_begin[kMaxOut] = {};
  int width[kMaxOut] = {};
  int trigger = 0;
  int pdl_wait = 0;
  int force_slow = 0;  // testing: always take the BF16-MMA path of the quantised modes
  unsigned long long* phase_times = nullptr;  // [CTA][16] timer stamps; written only by builds with -DQFG_PHASE_TIMES
  // plan
  int wn = 4, wk = 2, ks = 1, stages = 4, cluster = 1, gran = 16;
  int scales_l1 = 0;    // NVFP4 warp rings: copy the scale pieces through L1 (set where the CTA's shared memory leaves L1 room)
  int xpitch = 0;       // elements per x row in shared memory
  int ring_bytes = 0;   // stages * stage_bytes
  int stage_bytes = 0;
  int tile_row_bytes = 0;   // wn * bytes_per_warp
  int scale_row_bytes = 0;  // NVFP4: shared-memory bytes per row of the scale region
  // fused LM head (argmax over the BF16-rounded outputs of segment 0)
  int lm = 0;
  unsigned long long* lm_keys = nullptr;  // [kMaxRows] workspace, zero between calls
  unsigned int* lm_count = nullptr;       // workspace counter, zero between calls
  long long* lm_idx = nullptr;
  float* lm_val = nullptr;
  unsigned long long* lm_key_out = nullptr;
  long long lm_col_offset = 0;
  // Shared tail of the fused LM head.  When the 128-column groups of the vocabulary do not divide by the
  // CTA count (151936 = 1187 groups on 148 SMs), the `tail_groups` left-over groups are not given to a few
  // CTAs, which would then run 12 % longer than the rest: warps that have no columns of their own (the last
  // warp column of every CTA) each take one of `tail_split` slices of the K range of one left-over group,
  // store the FP32 partial sums to `lm_tail` ([group][slice][8 rows][128]), and the last CTA to arrive adds
  // the slices up in slice order.  `tail_stride` > 0: slice j of the groups * split runs in CTA j * tail_stride
  // (one per CTA, evenly spread: a CTA that hosts several runs that much longer than the rest); 0: the idle
  // warps take the slices in order, CTA by CTA (launches with fewer CTAs than slices).
  int tail_groups = 0;
  int tail_split = 1;
  int tail_stride = 0;
  float* lm_tail = nullptr;

  // SharedExpertDown (fuse != 0): x is replaced by swish_mul(x, x2) while it is staged, and the output is
  // routed + bf16(bf16(sum) * gate[m]) with gate[m] = bf16(sigmoid(bf16(dot(gx[m], gw)))).
  int fuse = 0;
  const uint16_t* x2 = nullptr;      // BF16 [M, K]
  const uint16_t* gx = nullptr;      // BF16 [M, gk]
  const uint16_t* gw = nullptr;      // BF16 [gk]
  const uint16_t* routed = nullptr;  // BF16 [M, N] or null
  int gk = 0;
  // Key exchange of the N-sharded LM head through peer memory (world > 1): xpeer[r] is rank r's buffer.
  int xworld = 1;
  int xrank = 0;
  int xspin = kExchangeSpin;              // iterations a thread waits for one word of a peer
  unsigned int* lm_status_out = nullptr;  // optional (host-mapped) word: 1 if a wait ran out in this call, else 0
  struct LmExchange* xpeer[8] = {};
};

// One rank's exchange buffer.  A word is (upper or lower half of a key) << 32 | call count of the writer, so
// its arrival validates itself.  Slots alternate with the parity of the call count, so a rank that is one
// call ahead never overwrites words a slower rank has not read yet.
struct LmExchange {
  unsigned long long words[2][8][kMaxRows][2];  // [parity][source rank][row][half]
  unsigned int epoch;                           // calls made by the owner
  unsigned int status;                          // 1 after a wait that ran out (until the host clears it)
  unsigned long long t_ready, t_sent, t_done;   // %globaltimer of the owner's last call: keys ready, stores issued, all words seen
};

constexpr int kMaxTailGroups = 8;
constexpr int kMaxTailSplit = 16;
constexpr size_t kLmHeaderBytes = 256;  // keys, counter, padding
constexpr size_t kLmTailBytes = static_cast<size_t>(kMaxTailGroups) * kMaxTailSplit * kMaxRows * 128 * 4;

// planner.cc
struct PlanInput {
  int K = 0;
  int nseg = 0;
  int n[kMaxSeg] = {};
  int mode = 0;
  int row_align = 16;  // min over segments of the alignment (16 / 8 / 4) of base and pitch
  int sm_count = 148;
  int max_rows = kMaxRows;
  // Co-resident clusters (CTAs for cluster == 1) of a launch shape on the current device, or null
  // when planning without a device (then a B200-like packing loss is assumed for clusters).
  int (*max_clusters)(int mode, int direct, int threads, size_t smem, int cluster) = nullptr;
  bool allow_tail = false;  // the call is a fused LM head whose workspace can hold the shared-tail partial sums
};
Plan ChoosePlan(const PlanInput& in);
// Applies "key=value,..." overrides (wn, wk, ks, stages, cluster, ctas, gran); returns false on a bad key.
bool ApplyPlanOverrides(const std::string& spec, const PlanInput& in, Plan* plan);
void FitRing(const PlanInput& in, int rows, Plan* plan);
// The decisions that follow the launch shape (`spec`: the override string): the shared tail of a fused LM head.
void FinishPlan(const PlanInput& in, const std::string& spec, Plan* plan);
// Decides Plan::tail for a fused LM head (see GemmParams::tail_groups); `forced`: the override gave a value.
void ChooseTail(const PlanInput& in, bool forced, Plan* plan);
void DistributeTiles(const PlanInput& in, int total_tiles, Plan* plan);
size_t SmemBytes(const Plan& plan, int mode, int rows, int K);
std::string DescribePlan(const Plan& plan, const PlanInput& in);

// skinny_gemm.cu
cudaError_t LaunchSkinnyGemm(int mode, GemmParams& p, const Plan& plan, cudaStream_t stream);
int DeviceSmCount();
cudaError_t ConfigureSkinnyGemmKernels();
int QueryMaxActiveClusters(int mode, int direct, int threads, size_t smem, int cluster);

// argmax_rows.cu
cudaError_t LaunchArgmaxRows(int dtype, const void* x, int64_t rows, int64_t vocab, int64_t* idx, float* val,
                             cudaStream_t stream);
cudaError_t LaunchLmheadCombine(const uint64_t* keys, int ranks, int64_t m, int64_t* idx, float* val,
                                cudaStream_t stream);

// capi.cc
int LmheadComputeWithWorkspace(const qfg_lmhead* op, const void* x, int64_t m, int64_t k, const qfg_tensor2d* weight,
                               int64_t n, int64_t col_offset, void* workspace, size_t workspace_bytes, int64_t* idx,
                               float* val, uint64_t* key, void* logits, void* stream,
                               const qfg_lmhead_exchange* exchange = nullptr, unsigned int* status_out = nullptr);
int SetLastError(int code, const char* message);

// dequant_bf16.cu
struct DequantParams {
  const uint8_t* w = nullptr;
  const float* w_scale = nullptr;
  int mode = 0;
  int K = 0;
  int N = 0;            // columns produced
  int row_stride = 0;   // logical columns of a stored row
  int col_offset = 0;
  int num_outs = 1;
  uint16_t* out[kMaxOut] = {};
  int col_begin[kMaxOut] = {};
  int width[kMaxOut] = {};
  int aligned = 1;      // vector loads are legal for every row
  int scale_vec = 0;    // set by LaunchDequant: w_scale can be read with 16-byte loads
};
cudaError_t LaunchDequant(const DequantParams& p, cudaStream_t stream);

// dense_gemm.cc: calls with more than `dense_rows` rows (an option of the node; 0 disables the branch).
// The defaults are where the branch starts to win on a B200 (K = 5120): BF16 weights need no dequantisation
// pass, so two streaming passes already lose (N = 2048: 37.7 us against 16.3); FP8 pays 48.5 us at N = 10240
// against 35 us per eight rows; NVFP4 pays 89 us at N = 17408, which three passes (105 us) exceed.
constexpr int DenseRowsDefault(int mode) { return mode == kNvfp4 ? 16 : 8; }
bool DenseEligible(const GemmParams& p);
void LaunchDenseGemm(int mode, const GemmParams& p, int64_t m, cudaStream_t stream);  // throws std::runtime_error

// untile_hc.cu
cudaError_t LaunchUntileHc(bool fp8, const void* w, void* out, const float* scale, int kind, cudaStream_t stream);

}  // namespace qfg

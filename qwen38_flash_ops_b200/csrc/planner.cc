// Launch planning for the streaming kernel: how many column tiles per weight, how many warps
// side by side, how deep the ring, how many CTAs split K.  The plan is a function of
// (K, segment widths, weight type, row alignment, SM count) only - the number of rows never
// enters, so a row is reduced in the same order whatever the batch (the property the reference
// states at src/fused_gemm/fused_gemm.cu:157-158).  The reference's H200 table (:132-156) is
// replaced by a rule that fills a B200: about two CTAs per SM, tiles at least 256 bytes wide per
// weight row where the shape allows it, K split across a cluster only as far as needed for that.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <sstream>

#include "qfg_internal.h"

namespace qfg {

namespace {

double BytesPerCol(int mode) { return mode == kBf16 ? 2.0 : mode == kFp8 ? 1.0 : 0.5; }

int Granule(int mode, int row_align, bool direct, int wide = 1) {
  const ModeGeom g = GeomOf(mode, direct ? wide : 1);
  if (direct && mode == kNvfp4) return 128;  // tiles are whole warp columns: aligned nibble chunks, scales in one 16-byte piece
  if (direct) return g.cols_per_thread;      // tiles are whole thread chunks
  const int cols_per_vec = static_cast<int>(row_align / BytesPerCol(mode));
  return std::max(g.cols_per_thread, cols_per_vec);
}

// The register-streaming kernel needs whole thread chunks and rows aligned to its load width.
bool DirectEligible(const PlanInput& in, int wide = 1) {
  const ModeGeom g = GeomOf(in.mode, wide);
  // BF16 / FP8 lanes copy their own 16 bytes; NVFP4 rows are copied as aligned 16-byte pieces
  // around chunks that may start 8 bytes off
  if (in.row_align < (in.mode == kNvfp4 ? 8 : 16)) return false;
  if (wide != 1) return false;  // the warp-ring kernel has one thread width
  for (int s = 0; s < in.nseg; ++s) {
    if (in.n[s] % (in.mode == kNvfp4 ? 128 : g.cols_per_thread) != 0) return false;
  }
  return true;
}

int MinTiles(const PlanInput& in, int max_cols, int gran) {
  int t = 0;
  for (int s = 0; s < in.nseg; ++s) {
    // a tile covers floor-or-ceil(granules / tiles) granules, so the widest tile must still fit
    const int granules = (in.n[s] + gran - 1) / gran;
    const int per_tile = std::max(1, max_cols / gran);
    t += (granules + per_tile - 1) / per_tile;
  }
  return t;
}

}  // namespace

// Ring depth and stage height for `rows` rows of x.  Neither changes which k-steps a warp
// accumulates (warp j of the wk warps always takes the k-steps congruent to j modulo wk, in
// increasing order), so unlike the rest of the plan they may depend on the row count.
void FitRing(const PlanInput& in, int rows, Plan* p) {
  const ModeGeom g = GeomOf(in.mode);
  if (p->direct) {
    // warp-private rings: as deep as the CTA's share of shared memory allows, at most 8 k-steps
    const int warps = p->warps();
    const int per_sm = p->tc ? 1 : std::max(1, (p->wide == 2 ? 16 : kMaxWarps) / warps);
    const size_t budget = static_cast<size_t>(220 * 1024) / per_sm;
    p->ks = 1;
    // the warp-ring kernel is compiled for rings of 8, 6 and 4 k-steps, the tcgen05 kernel for 6, 4 and 3
    static const int kDepths[] = {8, 6, 4, 3};
    // NVFP4 warp rings keep their scale bytes in L1: stay within the carve-out that leaves L1 room where a depth fits it
    const size_t want = (in.mode == kNvfp4 && !p->tc) ? std::min(budget, kL1FriendlySmem) : budget;
    for (int d : kDepths) {
      if (p->tc ? d == 8 : d == 3) continue;
      p->stages = d;
      if (SmemBytes(*p, in.mode, rows, in.K) <= want) break;
    }
    return;
  }
  const int tb = p->wn * g.bytes_per_warp + (in.mode == kNvfp4 ? (p->wn * 8 + 16 + 15) & ~15 : 0);
  // stages of about 8 KiB, ring of about 64 KiB
  p->ks = std::min(4, std::max(1, 8192 / (16 * p->wk * tb)));
  const int stage = 16 * p->wk * p->ks * tb;
  p->stages = std::min(8, std::max(3, 65536 / std::max(stage, 1)));
  // two CTAs per SM must fit
  while (p->stages > 3 && SmemBytes(*p, in.mode, rows, in.K) > 112 * 1024) --p->stages;
  while (p->ks > 1 && SmemBytes(*p, in.mode, rows, in.K) > 112 * 1024) --p->ks;
}

size_t SmemBytes(const Plan& plan, int mode, int rows, int K) {
  const ModeGeom g = GeomOf(mode, plan.direct ? plan.wide : 1);
  const int ksteps = (K + 15) / 16;
  const int kslice = ((ksteps + plan.cluster - 1) / plan.cluster) * 16;
  if (plan.tc) {
    // rings of the tensor-memory warps and of the mma.sync warps, reused for the partial sums; x as the
    // K-major MMA operand (256 bytes per k-step, one spare step that the 16-row instruction reads past the end)
    const int tnc = PlanMaxCols(plan, mode);
    const int red = (plan.wk + (plan.cluster > 1 ? 1 : 0)) * rows * tnc * 4;
    const int ring_raw = (plan.wn * plan.wk + plan.wk) * plan.stages * DirectSlotBytes(mode, 1);
    const int ring = (std::max(ring_raw, red) + 127) & ~127;
    const size_t total = static_cast<size_t>(ring) + static_cast<size_t>(kslice / 16 + 1) * 256;
    return std::max<size_t>(total, 120 * 1024);  // never two CTAs per SM: each allocates up to all of tensor memory
  }
  const int tb = plan.wn * g.bytes_per_warp;
  const int srb = mode == kNvfp4 ? (plan.wn * 8 + 16 + 15) & ~15 : 0;
  const int stage = (plan.rows_per_stage() * (tb + srb) + 127) & ~127;
  const int tnc = plan.wn * g.cols_per_warp;
  const int red = (plan.wk + (plan.cluster > 1 ? 1 : 0)) * rows * tnc * 4;
  const int direct_slot = RingSlotBytes(mode);
  const int ring_raw = plan.direct == 2 ? 0 : plan.direct ? plan.wn * plan.wk * plan.stages * direct_slot : plan.stages * stage;
  const int ring = (std::max(ring_raw, red) + 127) & ~127;
  const int xpitch = ((kslice + 63) & ~63) + 16;
  return static_cast<size_t>(ring) + static_cast<size_t>(rows) * xpitch * 2;
}

void DistributeTiles(const PlanInput& in, int total_tiles, Plan* plan) {
  const int max_cols = PlanMaxCols(*plan, in.mode);
  long long sum_n = 0;
  int min_t[kMaxSeg], given = 0;
  for (int s = 0; s < in.nseg; ++s) {
    sum_n += in.n[s];
    PlanInput one = in;
    one.nseg = 1;
    one.n[0] = in.n[s];
    min_t[s] = MinTiles(one, max_cols, plan->gran);
  }
  // proportional share, never below what the tile width requires, never above one tile per granule
  double frac[kMaxSeg];
  for (int s = 0; s < in.nseg; ++s) {
    const double share = static_cast<double>(total_tiles) * in.n[s] / static_cast<double>(sum_n);
    const int granules = (in.n[s] + plan->gran - 1) / plan->gran;
    int t = std::max(min_t[s], static_cast<int>(std::floor(share)));
    t = std::min(t, std::max(granules, 1));
    plan->tiles[s] = t;
    frac[s] = share - std::floor(share);
    given += t;
  }
  while (given < total_tiles) {
    int best = -1;
    for (int s = 0; s < in.nseg; ++s) {
      const int granules = (in.n[s] + plan->gran - 1) / plan->gran;
      if (plan->tiles[s] >= granules) continue;
      if (best < 0 || frac[s] > frac[best]) best = s;
    }
    if (best < 0) break;
    ++plan->tiles[best];
    frac[best] = -1.0;
    ++given;
    bool all_used = true;
    for (int s = 0; s < in.nseg; ++s) all_used = all_used && frac[s] < 0;
    if (all_used)
      for (int s = 0; s < in.nseg; ++s) frac[s] = static_cast<double>(in.n[s]) / static_cast<double>(sum_n);
  }
  for (int s = in.nseg; s < kMaxSeg; ++s) plan->tiles[s] = 0;
}

// Candidate launch shapes are scored by how much of the machine they keep busy:
//   lane efficiency  - columns a CTA can hold versus columns its tile actually has;
//   balance          - CTAs versus the resident CTA slots of whole waves (16 warps per SM);
//   pipeline length  - k-steps per warp, so that fill and drain of the load pipeline amortise;
//   row width        - contiguous bytes a CTA reads per weight row.
// Launch shapes measured best on B200 (148 SMs) for the decode GEMMs of the model this library
// serves; the counterpart of the reference's H200 table (src/fused_gemm/fused_gemm.cu:132-156).
// Every other shape, and these shapes on a different SM count, go through the scoring rule below.
struct TunedShape {
  int mode, K, nseg;
  int n[kMaxSeg];
  const char* spec;
};
const TunedShape kTunedB200[] = {
    {kBf16, 5120, 1, {5120, 0, 0, 0}, "direct=2,wn=1,wk=16,cluster=1,waves=1"},
    {kFp8, 5120, 3, {8192, 1024, 1024, 0}, "direct=2,wn=1,wk=16,cluster=1,ctas=148"},
    {kNvfp4, 5120, 2, {17408, 17408, 0, 0}, "direct=1,wide=1,wn=2,wk=8,cluster=1,ctas=136"},
    {kNvfp4, 17408, 1, {5120, 0, 0, 0}, "direct=1,wide=1,wn=2,wk=8,cluster=6,ctas=120"},
    {kNvfp4, 5120, 1, {151936, 0, 0, 0}, "direct=1,wide=1,wn=9,wk=2,cluster=1,waves=1"},
    // one eighth of that head where the split leaves 149 column groups: 30 tiles of five groups (one of four)
    // on 120 SMs beat the scored 32 uneven tiles on 128 (31.7 us against 33.1)
    {kNvfp4, 5120, 1, {19072, 0, 0, 0}, "direct=1,wide=1,wn=5,wk=4,cluster=4,ctas=120"},
};

Plan ChoosePlan(const PlanInput& in) {
  if (in.allow_tail && in.nseg == 1 && in.mode == kNvfp4 && in.n[0] % 128 == 0 && DirectEligible(in)) {
    // A fused LM head (or a shard of one) with at least four 128-column groups per SM: one CTA per SM with
    // `per` warp columns of its own and one more whose warps share the left-over groups (measured 7 % faster
    // than the scored plan on the 76032-column half shard, 10 % on the full 151936-column head).
    const int groups = in.n[0] / 128, per = groups / in.sm_count;
    if (per >= 4 && per + 1 <= 10 && groups - per * in.sm_count <= kMaxTailGroups) {
      char spec[96];
      std::snprintf(spec, sizeof(spec), "direct=1,wide=1,wn=%d,wk=%d,cluster=1,ctas=%d", per + 1, kMaxWarps / (per + 1), in.sm_count);
      Plan shared;
      if (ApplyPlanOverrides(spec, in, &shared)) return shared;
    }
  }
  if (in.sm_count == 148 && DirectEligible(in)) {
    for (const TunedShape& t : kTunedB200) {
      bool same = t.mode == in.mode && t.K == in.K && t.nseg == in.nseg;
      for (int s = 0; same && s < in.nseg; ++s) same = t.n[s] == in.n[s];
      Plan tuned;
      if (same && ApplyPlanOverrides(t.spec, in, &tuned)) return tuned;
    }
  }
  if ((in.mode == kBf16 || in.mode == kFp8) && DirectEligible(in)) {
    // BF16 / FP8 weights outside the table: the register-streaming kernel with one warp column per CTA beat
    // every warp-ring shape on the ten projection shapes of a K = 2560 model by 15-35 % (measured on a B200:
    // N from 320 to 16480, K from 320 to 10240).  K is split over the smallest cluster that gives every SM a
    // CTA (a warp column is 64 BF16 / 128 FP8 columns wide), as long as a warp keeps two k-steps or more.
    const ModeGeom g1 = GeomOf(in.mode, 1);
    long long total_n = 0;
    for (int s = 0; s < in.nseg; ++s) total_n += in.n[s];
    const int natural_tiles = static_cast<int>((total_n + g1.cols_per_warp - 1) / g1.cols_per_warp);
    const int ksteps = (in.K + 15) / 16;
    int cluster = 1;
    while (cluster < 8 && natural_tiles * cluster < in.sm_count * 7 / 8) cluster *= 2;
    int wk = (in.mode == kFp8 && cluster == 1) ? 16 : 8;
    while (cluster > 1 && ksteps < 2 * cluster * wk) cluster /= 2;
    // short K (32 to 64 k-steps, the SharedExpertDown class): the whole call is fixed phases, and a cluster
    // epilogue costs more than the idle SMs (640 x 2560: 5.6 us with sixteen warps and no cluster, 6.5 with two CTAs
    // per column tile; SharedExpertDown 8.4 against 10.3 us)
    if (ksteps >= 32 && ksteps <= 64) {
      cluster = 1;
      wk = 16;
    }
    char spec[96];
    std::snprintf(spec, sizeof(spec), "direct=2,wn=1,wk=%d,cluster=%d,waves=1", wk, cluster);
    Plan streaming;
    if (ApplyPlanOverrides(spec, in, &streaming)) return streaming;
  }
  if (in.mode == kNvfp4 && DirectEligible(in)) {
    // NVFP4 weights with no more 128-column groups than SMs: one group per CTA, sixteen warps sharing its K
    // range, and K split over the largest cluster (of a size that packs into a GPC) that the SM count allows.
    // Within 2 % of the best of 43 launch shapes on four such shapes (K 2560-6144, N 2560-17408), where the
    // scoring rule below was up to 20 % off.
    long long total_n = 0;
    for (int s = 0; s < in.nseg; ++s) total_n += in.n[s];
    const int groups = static_cast<int>(total_n / 128);
    const int ksteps = (in.K + 15) / 16;
    if (groups >= 1 && groups <= in.sm_count) {
      static const int kSizes[] = {8, 6, 4, 3, 2, 1};
      int cluster = 1;
      for (int c : kSizes) {
        if (c * groups <= in.sm_count && ksteps >= 2 * c * 16) {
          cluster = c;
          break;
        }
      }
      char spec[96];
      std::snprintf(spec, sizeof(spec), "direct=1,wide=1,wn=1,wk=16,cluster=%d,waves=1", cluster);
      Plan grouped;
      if (ApplyPlanOverrides(spec, in, &grouped)) return grouped;
    }
  }
  const double bpc = BytesPerCol(in.mode);
  long long sum_n = 0;
  for (int s = 0; s < in.nseg; ++s) sum_n += in.n[s];
  const bool direct = DirectEligible(in);
  const int ksteps = (in.K + 15) / 16;

  Plan best;
  double best_score = -1.0;
  for (int wide = 1; wide <= 2; ++wide) {
  if (wide == 2 && (in.mode != kNvfp4 || !DirectEligible(in, 2))) break;
  const ModeGeom g = GeomOf(in.mode, direct ? wide : 1);
  const int gran = Granule(in.mode, in.row_align, direct, wide);
  long long granules = 0;
  for (int s = 0; s < in.nseg; ++s) granules += (in.n[s] + gran - 1) / gran;
  const int max_warps = direct ? (wide == 2 ? 16 : kMaxWarps) : 8;
  const int max_wn = direct ? 10 : 8;
  for (int c = 1; c <= 8; c *= 2) {
    if (c > 1 && in.K / c < 256) continue;
    for (int wn = 1; wn <= max_wn; ++wn) {
      if (!direct && (wn & (wn - 1)) != 0) continue;                 // the ring's swizzle wants 2^n warps
      if (!direct && in.mode == kNvfp4 && wn < 2 && sum_n >= 256) continue;
      for (int wk = 1; wn * wk <= max_warps; ++wk) {
        if (!direct && (wk & (wk - 1)) != 0) continue;
        Plan p;
        p.wn = wn;
        p.wk = wk;
        p.cluster = c;
        p.gran = gran;
        p.direct = direct ? 1 : 0;
        p.wide = wide;
        p.ks = 1;
        p.stages = 3;
        // eight x rows must fit beside the partial sums, whatever the row count of a call
        const size_t smem = SmemBytes(p, in.mode, kMaxRows, in.K);
        if (smem > 200 * 1024 && c < 8) continue;
        const int per_sm = std::max(1, std::min(max_warps / (wn * wk), static_cast<int>((220 * 1024) / std::max<size_t>(smem, 1))));
        // clusters that can be resident at once: GPC boundaries cost a cluster launch some SMs
        int cluster_slots;
        if (in.max_clusters != nullptr) {
          cluster_slots = in.max_clusters(in.mode, p.direct * p.wide, wn * wk * 32, smem, c);
        } else {
          cluster_slots = c == 1 ? per_sm * in.sm_count : static_cast<int>(per_sm * in.sm_count * 0.89) / c;
        }
        if (cluster_slots < 1) continue;
        const int slots = cluster_slots * c;
        const int max_cols = wn * g.cols_per_warp;
        const int min_tiles = MinTiles(in, max_cols, gran);
        for (int waves = 1; waves <= 4; ++waves) {
          int tiles = std::max(min_tiles, waves * cluster_slots);
          tiles = static_cast<int>(std::min<long long>(tiles, std::max<long long>(granules, 1)));
          const int ctas = tiles * c;
          const int need = (tiles + cluster_slots - 1) / cluster_slots;
          const double balance = static_cast<double>(tiles) / (static_cast<double>(need) * cluster_slots) *
                                 std::min(1.0, static_cast<double>(slots) / (per_sm * in.sm_count));
          const double widest = std::ceil(static_cast<double>(granules) / tiles) * gran;
          const double lane_eff = std::min(1.0, (static_cast<double>(sum_n) / tiles) / max_cols) *
                                  ((static_cast<double>(sum_n) / tiles) / std::max(widest, 1.0));
          // 16 warps saturate an SM; a wide warp keeps twice the bytes in flight
          const double warps_per_sm = std::min(16.0, static_cast<double>(per_sm * wn * wk * wide));
          const double steps = static_cast<double>(ksteps) / c / wk / need;
          const double kfactor = std::min(1.0, steps / 12.0);
          const double row_bytes = (static_cast<double>(sum_n) / tiles) * bpc;
          const double rowfactor = std::sqrt(std::min(1.0, row_bytes / 128.0));
          double score = lane_eff * balance * (warps_per_sm / 16.0) * (0.5 + 0.5 * kfactor) * rowfactor;
          // wider threads fetch fewer partly used sectors and spend fewer instructions per weight
          if (wide == 2) score *= 0.9;  // measured: the wide warp pays off only where tiles are narrow and K is split
          // a second wave pays the per-CTA fixed costs (x staging, pipeline fill, epilogue) again
          score *= (1.0 - 0.015 * std::log2(static_cast<double>(c))) * std::pow(0.85, need - 1);
          if (score > best_score) {
            best_score = score;
            best = p;
            DistributeTiles(in, tiles, &best);
          }
          if (tiles == min_tiles && waves * cluster_slots <= min_tiles) break;
        }
      }
    }
  }
  }
  FitRing(in, in.max_rows, &best);
  return best;
}

bool ApplyPlanOverrides(const std::string& spec, const PlanInput& in, Plan* plan) {
  if (spec.empty()) return true;
  std::stringstream ss(spec);
  std::string item;
  int ctas = -1, waves = -1;
  bool ring_given = false, wide_given = false, shape_given = false, gran_given = false;
  while (std::getline(ss, item, ',')) {
    const size_t eq = item.find('=');
    if (eq == std::string::npos) return false;
    const std::string key = item.substr(0, eq);
    const int val = std::atoi(item.substr(eq + 1).c_str());
    if (key == "wn") { plan->wn = val; shape_given = true; }
    else if (key == "wk") { plan->wk = val; shape_given = true; }
    else if (key == "ks") { plan->ks = val; ring_given = true; }
    else if (key == "stages") { plan->stages = val; ring_given = true; }
    else if (key == "cluster") plan->cluster = val;
    else if (key == "ctas") ctas = val;
    else if (key == "waves") waves = val;
    else if (key == "gran") { plan->gran = val; gran_given = true; }
    else if (key == "direct") plan->direct = val;
    else if (key == "wide") { plan->wide = val; wide_given = true; }
    else if (key == "tc") plan->tc = val != 0 ? 1 : 0;
    else if (key == "tail") plan->tail = val;
    else return false;
  }
  auto pow2 = [](int v) { return v > 0 && (v & (v - 1)) == 0; };
  if (shape_given && !wide_given) plan->wide = 1;  // a warp shape without a width means the 128-column warp
  if (plan->wide != 1 && plan->wide != 2) return false;
  if (plan->direct == 0 || in.mode != kNvfp4) plan->wide = 1;
  if (plan->direct != 0 && !DirectEligible(in, plan->wide)) return false;
  if (plan->tc != 0) {
    // tensor-memory budget: 64 accumulator columns per 512-column group and 3 x 32 per warpgroup
    if (in.mode != kNvfp4 || plan->direct == 0 || plan->wide != 1 || plan->wn % 4 != 0 ||
        (plan->wn / 4) * (64 + plan->wk * 96) > 512 || plan->warps() > 20 || plan->wn * plan->wk / 4 > 8) {
      return false;
    }
  }
  if (plan->direct != 0 && ring_given) {
    const int d = plan->stages;
    if (plan->tc != 0 ? (d != 3 && d != 4 && d != 6) : (d != 4 && d != 6 && d != 8)) return false;
  }
  // 2 = register streaming (BF16 / FP8, at most 16 warps)
  if (plan->direct == 2 && (in.mode == kNvfp4 || plan->wn * plan->wk > 16)) return false;
  plan->direct = plan->direct == 2 ? 2 : plan->direct != 0 ? 1 : 0;
  if (plan->direct == 0 && plan->gran < Granule(in.mode, in.row_align, false)) plan->gran = Granule(in.mode, in.row_align, false);
  if ((plan->direct == 0 && (!pow2(plan->wn) || !pow2(plan->wk) || plan->wn * plan->wk > 8)) || plan->wn < 1 || plan->wk < 1 ||
      plan->warps() > (plan->wide == 2 ? 16 : kMaxWarps) || plan->wn > 12 || plan->ks < 1 || plan->ks > 8 ||
      plan->stages < 2 || plan->stages > 8 || plan->cluster < 1 || plan->cluster > 8) {
    return false;
  }
  // the column granule belongs to the kernel: an override that changes the kernel takes that kernel's granule
  if (!gran_given || plan->gran % Granule(in.mode, in.row_align, plan->direct != 0, plan->wide) != 0)
    plan->gran = Granule(in.mode, in.row_align, plan->direct != 0, plan->wide);
  if (!ring_given) FitRing(in, in.max_rows, plan);
  const ModeGeom g = GeomOf(in.mode, plan->direct ? plan->wide : 1);
  int total = ctas > 0 ? std::max(1, ctas / plan->cluster) : 0;
  if (waves > 0) {
    // as many tiles as `waves` full waves of co-resident clusters hold
    // tiles must not depend on the rows of the call: size the launch as for a full row block
    Plan full = *plan;
    if (!ring_given) FitRing(in, kMaxRows, &full);
    const size_t smem = SmemBytes(full, in.mode, kMaxRows, in.K);
    const int per_sm = std::max(1, std::min(kMaxWarps / (plan->wn * plan->wk), static_cast<int>((220 * 1024) / std::max<size_t>(smem, 1))));
    int cluster_slots;
    if (in.max_clusters != nullptr) {
      cluster_slots = in.max_clusters(in.mode, plan->tc ? 3 : plan->direct == 2 ? 4 : plan->direct * plan->wide, plan->threads(), smem,
                                      plan->cluster);
    } else {
      cluster_slots = plan->cluster == 1 ? per_sm * in.sm_count : static_cast<int>(per_sm * in.sm_count * 0.89) / plan->cluster;
    }
    total = std::max(1, waves * cluster_slots);
  }
  const int min_tiles = MinTiles(in, PlanMaxCols(*plan, in.mode), plan->gran);
  if (total == 0) {
    total = 0;
    for (int s = 0; s < in.nseg; ++s) total += plan->tiles[s];
  }
  DistributeTiles(in, std::max(total, min_tiles), plan);
  return true;
}

// The shared tail needs: one NVFP4 weight of whole 128-column groups on the direct kernel with 128-column warps,
// no K split across CTAs (all CTAs must stage the same x), a workspace for the partial sums, and a warp
// column without columns of its own in every CTA.
void ChooseTail(const PlanInput& in, bool forced, Plan* plan) {
  const int want = plan->tail;
  plan->tail = 0;
  if (!in.allow_tail || in.nseg != 1 || in.mode != kNvfp4 || !plan->direct || plan->tc || plan->wide != 1 ||
      plan->cluster != 1 || in.n[0] % 128 != 0) {
    return;
  }
  const int groups = in.n[0] / 128, ctas = plan->tiles[0];
  if (ctas < 1) return;
  const int per = groups / ctas;
  int tail = groups - per * ctas;
  if (forced) tail = want;  // tests: any count that leaves whole groups per CTA
  if (tail < 1 || tail > kMaxTailGroups || tail >= groups || (groups - tail) % ctas != 0) return;
  if ((groups - tail) / ctas > plan->wn - 1) return;
  if (tail > ctas * plan->wk) return;  // every left-over group needs an idle warp of its own
  plan->tail = tail;
}

void FinishPlan(const PlanInput& in, const std::string& spec, Plan* plan) {
  ChooseTail(in, spec.find("tail=") != std::string::npos, plan);
}

std::string DescribePlan(const Plan& plan, const PlanInput& in) {
  char buf[256];
  int tiles = 0;
  for (int s = 0; s < in.nseg; ++s) tiles += plan.tiles[s];
  std::snprintf(buf, sizeof(buf),
                "direct=%d,tc=%d,tail=%d,wide=%d,wn=%d,wk=%d,ks=%d,stages=%d,cluster=%d,gran=%d,tiles=%d,ctas=%d,threads=%d,smem=%zu",
                plan.direct, plan.tc, plan.tail, plan.wide, plan.wn, plan.wk, plan.ks, plan.stages, plan.cluster, plan.gran, tiles,
                tiles * plan.cluster, plan.threads(),
                SmemBytes(plan, in.mode, in.max_rows, in.K));
  return buf;
}

}  // namespace qfg

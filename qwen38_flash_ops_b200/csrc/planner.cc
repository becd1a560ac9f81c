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

int Granule(int mode, int row_align) {
  const ModeGeom g = GeomOf(mode);
  const int cols_per_vec = static_cast<int>(row_align / BytesPerCol(mode));
  return std::max(g.cols_per_thread, cols_per_vec);
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
  const int tb = p->wn * g.bytes_per_warp + (in.mode == kNvfp4 ? p->wn * 8 + 16 : 0);
  // stages of about 8 KiB, ring of about 64 KiB
  p->ks = std::min(4, std::max(1, 8192 / (16 * p->wk * tb)));
  const int stage = 16 * p->wk * p->ks * tb;
  p->stages = std::min(8, std::max(3, 65536 / std::max(stage, 1)));
  // two CTAs per SM must fit
  while (p->stages > 3 && SmemBytes(*p, in.mode, rows, in.K) > 112 * 1024) --p->stages;
  while (p->ks > 1 && SmemBytes(*p, in.mode, rows, in.K) > 112 * 1024) --p->ks;
}

size_t SmemBytes(const Plan& plan, int mode, int rows, int K) {
  const ModeGeom g = GeomOf(mode);
  const int tb = plan.wn * g.bytes_per_warp;
  const int srb = mode == kNvfp4 ? plan.wn * 8 + 16 : 0;
  const int stage = (plan.rows_per_stage() * (tb + srb) + 127) & ~127;
  const int tnc = plan.wn * g.cols_per_warp;
  const int red = (plan.wk + (plan.cluster > 1 ? 1 : 0)) * rows * tnc * 4;
  const int ring = (std::max(plan.stages * stage, red) + 127) & ~127;
  const int ksteps = (K + 15) / 16;
  const int kslice = ((ksteps + plan.cluster - 1) / plan.cluster) * 16;
  const int xpitch = ((kslice + 63) & ~63) + 16;
  return static_cast<size_t>(ring) + static_cast<size_t>(rows) * xpitch * 2;
}

void DistributeTiles(const PlanInput& in, int total_tiles, Plan* plan) {
  const ModeGeom g = GeomOf(in.mode);
  const int max_cols = plan->wn * g.cols_per_warp;
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

Plan ChoosePlan(const PlanInput& in) {
  const ModeGeom g = GeomOf(in.mode);
  const double bpc = BytesPerCol(in.mode);
  const int target = 2 * in.sm_count;
  long long sum_n = 0;
  for (int s = 0; s < in.nseg; ++s) sum_n += in.n[s];
  const int gran = Granule(in.mode, in.row_align);

  Plan best;
  double best_score = -1.0;
  for (int c = 1; c <= 8; c *= 2) {
    if (c > 1 && in.K / c < 256) continue;
    for (int wn = 1; wn <= 8; wn *= 2) {
      if (in.mode == kNvfp4 && wn < 2 && sum_n >= 256) continue;  // 64-byte rows defeat the swizzle
      Plan p;
      p.wn = wn;
      p.wk = 8 / wn;
      p.cluster = c;
      p.gran = gran;
      // the K slice of eight x rows must fit beside a minimal ring, whatever the row count of a call
      {
        Plan probe = p;
        probe.ks = 1;
        probe.stages = 3;
        if (c < 8 && SmemBytes(probe, in.mode, kMaxRows, in.K) > 200 * 1024) continue;
      }
      const int max_cols = wn * g.cols_per_warp;
      const int min_tiles = MinTiles(in, max_cols, gran);
      int tiles = std::max(min_tiles, target / c);
      long long granules = 0;
      for (int s = 0; s < in.nseg; ++s) granules += (in.n[s] + gran - 1) / gran;
      tiles = static_cast<int>(std::min<long long>(tiles, std::max<long long>(granules, 1)));
      const int ctas = tiles * c;
      const double width = static_cast<double>(sum_n) / tiles;
      const double row_bytes = width * bpc;
      const double lane_eff = static_cast<double>(sum_n) / (static_cast<double>(tiles) * max_cols);
      const int waves = (ctas + target - 1) / target;
      const double balance = static_cast<double>(ctas) / (static_cast<double>(waves) * target);
      const double fill = std::min(1.0, static_cast<double>(ctas) / target);
      double score = std::min(1.0, row_bytes / 256.0) * (0.5 + 0.5 * lane_eff) * balance * fill;
      score *= 1.0 - 0.02 * std::log2(static_cast<double>(c));
      if (waves > 1) score *= 0.8;
      if (score > best_score) {
        best_score = score;
        best = p;
        DistributeTiles(in, tiles, &best);
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
  int ctas = -1;
  bool ring_given = false;
  while (std::getline(ss, item, ',')) {
    const size_t eq = item.find('=');
    if (eq == std::string::npos) return false;
    const std::string key = item.substr(0, eq);
    const int val = std::atoi(item.substr(eq + 1).c_str());
    if (key == "wn") plan->wn = val;
    else if (key == "wk") plan->wk = val;
    else if (key == "ks") { plan->ks = val; ring_given = true; }
    else if (key == "stages") { plan->stages = val; ring_given = true; }
    else if (key == "cluster") plan->cluster = val;
    else if (key == "ctas") ctas = val;
    else if (key == "gran") plan->gran = val;
    else return false;
  }
  auto pow2 = [](int v) { return v > 0 && (v & (v - 1)) == 0; };
  if (!pow2(plan->wn) || !pow2(plan->wk) || plan->wn * plan->wk > 8 || plan->ks < 1 || plan->ks > 8 ||
      plan->stages < 2 || plan->stages > 9 || plan->cluster < 1 || plan->cluster > 8 || !pow2(plan->cluster)) {
    return false;
  }
  if (plan->gran % Granule(in.mode, in.row_align) != 0) return false;
  if (!ring_given) FitRing(in, in.max_rows, plan);
  const ModeGeom g = GeomOf(in.mode);
  int total = ctas > 0 ? std::max(1, ctas / plan->cluster) : 0;
  const int min_tiles = MinTiles(in, plan->wn * g.cols_per_warp, plan->gran);
  if (total == 0) {
    total = 0;
    for (int s = 0; s < in.nseg; ++s) total += plan->tiles[s];
  }
  DistributeTiles(in, std::max(total, min_tiles), plan);
  return true;
}

std::string DescribePlan(const Plan& plan, const PlanInput& in) {
  char buf[256];
  int tiles = 0;
  for (int s = 0; s < in.nseg; ++s) tiles += plan.tiles[s];
  std::snprintf(buf, sizeof(buf),
                "wn=%d,wk=%d,ks=%d,stages=%d,cluster=%d,gran=%d,tiles=%d,ctas=%d,threads=%d,smem=%zu", plan.wn,
                plan.wk, plan.ks, plan.stages, plan.cluster, plan.gran, tiles, tiles * plan.cluster, plan.threads(),
                SmemBytes(plan, in.mode, in.max_rows, in.K));
  return buf;
}

}  // namespace qfg

// Native host-side runtime pieces (C++): memory arenas, the paged-KV block allocator, MoE token grouping and the
// grouped-GEMM planner, plus CPU reference implementations (router, logits processing, weight de-quantization,
// 2:4 pruning) that the tests use as an independent oracle for the CUDA kernels.
//
// Parity: reference cpp/src/pool.cpp + buffer_manager.cpp (sub-allocating heap with priority eviction, pin/unpin,
// transient ring with O(1) reset), cpp/src/gemm_dispatch.cpp (mixed bit-width batch planner), cpp/src/moe_manager.mm
// (stable token grouping + imbalance metrics), cpp/src/moe_router_dispatch.cpp (CPU router: GEMV + top-k),
// metal_marlin/cpp/logits_ops.hpp (temperature / softmax / top-k / top-p / repetition penalty),
// metal_marlin/utils/cpu_dequant.cpp (FP4 / INT4 / NF4 / INT8 / FP8 de-quantization), cpp/src/weights_ops.cpp (2:4).
// The arenas manage OFFSETS inside a slab the caller owns (a torch tensor on the GPU, pinned host memory, or a
// symmetric-memory buffer), so the same code serves device, pinned and peer-mapped heaps and never calls an allocator
// on the request path.
#include <torch/library.h>
#include <torch/torch.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <map>
#include <mutex>
#include <numeric>
#include <unordered_map>
#include <vector>

namespace {

using at::Tensor;

// ------------------------------------------------------------------------------------------------ arena
struct Block {
  int64_t size;
  bool free;
  bool pinned;
  int priority;
  int64_t last_use;
};

struct Arena {
  int64_t capacity, alignment, clock = 0, peak = 0, used = 0, n_alloc = 0, n_evict = 0;
  std::map<int64_t, Block> blocks;   // offset -> block, covering [0, capacity) without gaps

  Arena(int64_t cap, int64_t align) : capacity(cap), alignment(align) { blocks[0] = Block{cap, true, false, 0, 0}; }

  int64_t round(int64_t n) const { return (n + alignment - 1) / alignment * alignment; }

  void coalesce(std::map<int64_t, Block>::iterator it) {
    auto nx = std::next(it);
    if (nx != blocks.end() && nx->second.free) {
      it->second.size += nx->second.size;
      blocks.erase(nx);
    }
    if (it != blocks.begin()) {
      auto pv = std::prev(it);
      if (pv->second.free) {
        pv->second.size += it->second.size;
        blocks.erase(it);
      }
    }
  }

  int64_t try_alloc(int64_t need, int priority) {
    auto best = blocks.end();
    for (auto it = blocks.begin(); it != blocks.end(); ++it)
      if (it->second.free && it->second.size >= need && (best == blocks.end() || it->second.size < best->second.size)) best = it;
    if (best == blocks.end()) return -1;
    const int64_t off = best->first, rest = best->second.size - need;
    best->second = Block{need, false, false, priority, ++clock};
    if (rest > 0) blocks[off + need] = Block{rest, true, false, 0, 0};
    used += need;
    peak = std::max(peak, used);
    ++n_alloc;
    return off;
  }

  void release(int64_t off) {
    auto it = blocks.find(off);
    TORCH_CHECK(it != blocks.end() && !it->second.free, "arena: free of an offset that is not allocated: ", off);
    used -= it->second.size;
    it->second.free = true;
    it->second.pinned = false;
    coalesce(it);
  }

  // Best fit; when nothing fits, evict unpinned blocks of priority <= `priority` (lowest priority, then least recently
  // used first) until the request fits.  Evicted offsets are appended to `evicted` so the owner can drop its handles.
  int64_t alloc(int64_t nbytes, int priority, bool allow_evict, std::vector<int64_t>& evicted) {
    const int64_t need = round(std::max<int64_t>(nbytes, 1));
    int64_t off = try_alloc(need, priority);
    while (off < 0 && allow_evict) {
      auto victim = blocks.end();
      for (auto it = blocks.begin(); it != blocks.end(); ++it) {
        const Block& b = it->second;
        if (b.free || b.pinned || b.priority > priority) continue;
        if (victim == blocks.end() || b.priority < victim->second.priority ||
            (b.priority == victim->second.priority && b.last_use < victim->second.last_use))
          victim = it;
      }
      if (victim == blocks.end()) break;
      evicted.push_back(victim->first);
      ++n_evict;
      release(victim->first);
      off = try_alloc(need, priority);
    }
    return off;
  }

  // Slide every movable (unpinned) live block towards offset 0, closing the holes in front of it; pinned blocks stay
  // where they are and split the arena into segments that are compacted separately.  Returns (old offset, new offset,
  // size) triples in ascending order of the old offset: moving the bytes in that order with memmove semantics is safe.
  std::vector<int64_t> compact() {
    std::vector<int64_t> moves;
    std::map<int64_t, Block> out;
    int64_t cursor = 0;      // next free byte of the current segment
    auto flush_gap = [&](int64_t upto) {
      if (upto > cursor) out[cursor] = Block{upto - cursor, true, false, 0, 0};
    };
    for (auto& kv : blocks) {
      const Block& b = kv.second;
      if (b.free) continue;
      if (b.pinned) {
        flush_gap(kv.first);
        out[kv.first] = b;
        cursor = kv.first + b.size;
      } else {
        if (kv.first != cursor) {
          moves.push_back(kv.first);
          moves.push_back(cursor);
          moves.push_back(b.size);
        }
        out[cursor] = b;
        cursor += b.size;
      }
    }
    flush_gap(capacity);
    blocks.swap(out);
    return moves;
  }

  double fragmentation() const {
    int64_t free_total = 0, largest = 0;
    for (auto& kv : blocks)
      if (kv.second.free) {
        free_total += kv.second.size;
        largest = std::max(largest, kv.second.size);
      }
    return free_total ? 1.0 - (double)largest / (double)free_total : 0.0;
  }
};

std::mutex g_mu;
std::unordered_map<int64_t, Arena> g_arenas;
int64_t g_next_handle = 1;

int64_t arena_create(int64_t capacity, int64_t alignment) {
  TORCH_CHECK(capacity > 0 && alignment > 0 && (alignment & (alignment - 1)) == 0, "arena: bad capacity / alignment");
  std::lock_guard<std::mutex> lock(g_mu);
  g_arenas.emplace(g_next_handle, Arena(capacity, alignment));
  return g_next_handle++;
}
void arena_destroy(int64_t h) {
  std::lock_guard<std::mutex> lock(g_mu);
  g_arenas.erase(h);
}
Arena& arena_get(int64_t h) {
  auto it = g_arenas.find(h);
  TORCH_CHECK(it != g_arenas.end(), "arena: unknown handle ", h);
  return it->second;
}
// returns [offset, evicted offsets...]; offset -1 = out of memory
std::vector<int64_t> arena_alloc(int64_t h, int64_t nbytes, int64_t priority, bool allow_evict) {
  std::lock_guard<std::mutex> lock(g_mu);
  std::vector<int64_t> ev;
  const int64_t off = arena_get(h).alloc(nbytes, (int)priority, allow_evict, ev);
  ev.insert(ev.begin(), off);
  return ev;
}
void arena_free(int64_t h, int64_t off) {
  std::lock_guard<std::mutex> lock(g_mu);
  arena_get(h).release(off);
}
void arena_pin(int64_t h, int64_t off, bool pinned) {
  std::lock_guard<std::mutex> lock(g_mu);
  auto& a = arena_get(h);
  auto it = a.blocks.find(off);
  TORCH_CHECK(it != a.blocks.end() && !it->second.free, "arena: pin of an offset that is not allocated");
  it->second.pinned = pinned;
}
void arena_touch(int64_t h, int64_t off) {
  std::lock_guard<std::mutex> lock(g_mu);
  auto& a = arena_get(h);
  auto it = a.blocks.find(off);
  if (it != a.blocks.end() && !it->second.free) it->second.last_use = ++a.clock;
}
// [capacity, used, peak, n_alloc, n_evict, n_blocks, largest_free, fragmentation * 1e6]
std::vector<int64_t> arena_compact(int64_t h) {
  std::lock_guard<std::mutex> lk(g_mu);
  return arena_get(h).compact();
}
std::vector<int64_t> arena_stats(int64_t h) {
  std::lock_guard<std::mutex> lock(g_mu);
  auto& a = arena_get(h);
  int64_t largest = 0;
  for (auto& kv : a.blocks)
    if (kv.second.free) largest = std::max(largest, kv.second.size);
  return {a.capacity, a.used, a.peak, a.n_alloc, a.n_evict, (int64_t)a.blocks.size(), largest, (int64_t)(a.fragmentation() * 1e6)};
}

// ------------------------------------------------------------------------------------------------ MoE grouping / planner
// Stable counting sort of (token, slot) pairs by expert.  ids int32/int64 [T, k] (negative = dropped).  Returns
// (order int64 [n_valid], offsets int64 [E + 1], counts int64 [E]).
std::tuple<Tensor, Tensor, Tensor> cpu_group_tokens(const Tensor& ids, int64_t num_experts) {
  auto flat = ids.to(at::kLong).reshape({-1}).contiguous();
  const int64_t n = flat.numel();
  const int64_t* p = flat.data_ptr<int64_t>();
  auto counts = at::zeros({num_experts}, at::kLong);
  int64_t* c = counts.data_ptr<int64_t>();
  for (int64_t i = 0; i < n; ++i)
    if (p[i] >= 0 && p[i] < num_experts) ++c[p[i]];
  auto offsets = at::zeros({num_experts + 1}, at::kLong);
  int64_t* o = offsets.data_ptr<int64_t>();
  for (int64_t e = 0; e < num_experts; ++e) o[e + 1] = o[e] + c[e];
  auto order = at::empty({o[num_experts]}, at::kLong);
  int64_t* ord = order.data_ptr<int64_t>();
  std::vector<int64_t> cur(o, o + num_experts);
  for (int64_t i = 0; i < n; ++i)
    if (p[i] >= 0 && p[i] < num_experts) ord[cur[p[i]]++] = i;
  return {order, offsets, counts};
}

// Grouped-GEMM plan for experts of mixed bit widths: experts with work are grouped by bit width (one launch per
// group), each expert's rows cut into token tiles.  Returns int64 [n_tiles, 5]: (group, bits, expert, first_row, rows),
// sorted by (bits, expert).
Tensor plan_grouped_gemm(const Tensor& counts, const Tensor& offsets, const Tensor& expert_bits, int64_t token_tile) {
  TORCH_CHECK(token_tile > 0);
  auto c = counts.to(at::kLong).contiguous(), o = offsets.to(at::kLong).contiguous(), b = expert_bits.to(at::kLong).contiguous();
  const int64_t E = c.numel();
  std::vector<int64_t> experts(E);
  std::iota(experts.begin(), experts.end(), 0);
  const int64_t* bp = b.data_ptr<int64_t>();
  std::stable_sort(experts.begin(), experts.end(), [&](int64_t x, int64_t y) { return bp[x] < bp[y]; });
  std::vector<int64_t> rows;
  int64_t group = -1, last_bits = -1;
  for (int64_t e : experts) {
    const int64_t n = c.data_ptr<int64_t>()[e];
    if (n == 0) continue;
    if (bp[e] != last_bits) {
      ++group;
      last_bits = bp[e];
    }
    for (int64_t r = 0; r < n; r += token_tile) {
      rows.insert(rows.end(), {group, bp[e], e, o.data_ptr<int64_t>()[e] + r, std::min(token_tile, n - r)});
    }
  }
  auto out = at::empty({(int64_t)rows.size() / 5, 5}, at::kLong);
  std::copy(rows.begin(), rows.end(), out.data_ptr<int64_t>());
  return out;
}

// ------------------------------------------------------------------------------------------------ CPU references
const float kE2M1[16] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f, -0.f, -.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};

// codes uint8 [out, in] (one FP4 code per byte), scales fp16/fp32 [out, in / gs] -> fp32 [out, in]
Tensor cpu_dequant_fp4(const Tensor& codes, const Tensor& scales) {
  auto c = codes.contiguous();
  auto s = scales.to(at::kFloat).contiguous();
  const int64_t out_f = c.size(0), in_f = c.size(1), ng = s.size(1), gs = in_f / ng;
  auto w = at::empty({out_f, in_f}, at::kFloat);
  const uint8_t* cp = c.data_ptr<uint8_t>();
  const float* sp = s.data_ptr<float>();
  float* wp = w.data_ptr<float>();
  for (int64_t o = 0; o < out_f; ++o)
    for (int64_t i = 0; i < in_f; ++i) wp[o * in_f + i] = kE2M1[cp[o * in_f + i] & 15] * sp[o * ng + i / gs];
  return w;
}

// generic codebook: w = (lut[code] - zero) * scale
Tensor cpu_dequant_codebook(const Tensor& codes, const Tensor& scales, const c10::optional<Tensor>& zeros, const Tensor& lut) {
  auto c = codes.contiguous();
  auto s = scales.to(at::kFloat).contiguous();
  auto l = lut.to(at::kFloat).contiguous();
  Tensor z;
  if (zeros.has_value() && zeros->defined()) z = zeros->to(at::kFloat).contiguous();
  const int64_t out_f = c.size(0), in_f = c.size(1), ng = s.size(1), gs = in_f / ng;
  auto w = at::empty({out_f, in_f}, at::kFloat);
  for (int64_t o = 0; o < out_f; ++o)
    for (int64_t i = 0; i < in_f; ++i) {
      const float zp = z.defined() ? z.data_ptr<float>()[o * ng + i / gs] : 0.f;
      w.data_ptr<float>()[o * in_f + i] = (l.data_ptr<float>()[c.data_ptr<uint8_t>()[o * in_f + i]] - zp) * s.data_ptr<float>()[o * ng + i / gs];
    }
  return w;
}

// Router: logits = x W^T (fp32), scoring 0 = softmax, 1 = sigmoid (+ bias for the choice only), top-k, optional
// renormalisation, routed scale.  Returns (ids int32 [T, k], weights fp32 [T, k]).
std::tuple<Tensor, Tensor> cpu_router_topk(const Tensor& x, const Tensor& w, const c10::optional<Tensor>& bias, int64_t topk,
                                           int64_t scoring, bool renorm, double routed_scale) {
  auto xf = x.to(at::kFloat).contiguous(), wf = w.to(at::kFloat).contiguous();
  const int64_t T = xf.size(0), K = xf.size(1), E = wf.size(0);
  Tensor bf;
  if (bias.has_value() && bias->defined()) bf = bias->to(at::kFloat).contiguous();
  auto ids = at::empty({T, topk}, at::kInt);
  auto wts = at::empty({T, topk}, at::kFloat);
  std::vector<float> score(E), choice(E);
  std::vector<int> idx(E);
  for (int64_t t = 0; t < T; ++t) {
    float mx = -INFINITY;
    for (int64_t e = 0; e < E; ++e) {
      double acc = 0;
      const float *xr = xf.data_ptr<float>() + t * K, *wr = wf.data_ptr<float>() + e * K;
      for (int64_t k = 0; k < K; ++k) acc += (double)xr[k] * wr[k];
      score[e] = (float)acc;
      mx = std::max(mx, score[e]);
    }
    if (scoring == 0) {
      double sum = 0;
      for (int64_t e = 0; e < E; ++e) sum += (score[e] = std::exp(score[e] - mx));
      for (int64_t e = 0; e < E; ++e) score[e] = (float)(score[e] / sum);
    } else {
      for (int64_t e = 0; e < E; ++e) score[e] = 1.f / (1.f + std::exp(-score[e]));
    }
    for (int64_t e = 0; e < E; ++e) choice[e] = score[e] + (bf.defined() ? bf.data_ptr<float>()[e] : 0.f);
    std::iota(idx.begin(), idx.end(), 0);
    std::partial_sort(idx.begin(), idx.begin() + topk, idx.end(),
                      [&](int a, int b) { return choice[a] > choice[b] || (choice[a] == choice[b] && a < b); });
    double tot = 0;
    for (int64_t j = 0; j < topk; ++j) tot += score[idx[j]];
    for (int64_t j = 0; j < topk; ++j) {
      ids.data_ptr<int>()[t * topk + j] = idx[j];
      float v = score[idx[j]];
      if (renorm) v = (float)(v / (tot + 1e-20));
      wts.data_ptr<float>()[t * topk + j] = v * (float)routed_scale;
    }
  }
  return {ids, wts};
}

// Logits processing in the sampler's order: repetition penalty -> temperature -> top-k -> softmax -> top-p -> min-p ->
// renormalise.  Returns the probability vector fp32 [B, V].
Tensor cpu_logits_process(const Tensor& logits, double temperature, int64_t top_k, double top_p, double min_p, double rep_penalty,
                          const c10::optional<Tensor>& history) {
  auto lg = logits.to(at::kFloat).contiguous().clone();
  const int64_t B = lg.size(0), V = lg.size(1);
  Tensor hist;
  if (history.has_value() && history->defined()) hist = history->to(at::kLong).contiguous();
  for (int64_t b = 0; b < B; ++b) {
    float* r = lg.data_ptr<float>() + b * V;
    if (hist.defined() && rep_penalty != 1.0) {
      std::vector<char> seen(V, 0);
      for (int64_t j = 0; j < hist.size(1); ++j) {
        const int64_t t = hist.data_ptr<int64_t>()[b * hist.size(1) + j];
        if (t >= 0 && t < V && !seen[t]) {
          seen[t] = 1;
          r[t] = r[t] > 0 ? (float)(r[t] / rep_penalty) : (float)(r[t] * rep_penalty);
        }
      }
    }
    if (temperature > 0)
      for (int64_t i = 0; i < V; ++i) r[i] = (float)(r[i] / temperature);
    std::vector<int64_t> order(V);
    std::iota(order.begin(), order.end(), 0);
    std::sort(order.begin(), order.end(), [&](int64_t a, int64_t c) { return r[a] > r[c] || (r[a] == r[c] && a < c); });
    int64_t keep = (top_k > 0 && top_k < V) ? top_k : V;
    if (temperature <= 0) keep = 1;
    const float mx = r[order[0]];
    std::vector<double> p(V, 0.0);
    double sum = 0;
    for (int64_t j = 0; j < keep; ++j) sum += (p[order[j]] = std::exp((double)r[order[j]] - mx));
    for (int64_t j = 0; j < keep; ++j) p[order[j]] /= sum;
    if (top_p < 1.0) {
      double cum = 0;
      int64_t cut = keep;
      for (int64_t j = 0; j < keep; ++j) {
        cum += p[order[j]];
        if (cum >= top_p) {
          cut = j + 1;
          break;
        }
      }
      for (int64_t j = cut; j < keep; ++j) p[order[j]] = 0;
      keep = cut;
    }
    if (min_p > 0) {
      const double thr = min_p * p[order[0]];
      for (int64_t j = 0; j < keep; ++j)
        if (p[order[j]] < thr) p[order[j]] = 0;
    }
    double tot = 0;
    for (int64_t i = 0; i < V; ++i) tot += p[i];
    for (int64_t i = 0; i < V; ++i) r[i] = (float)(p[i] / tot);
  }
  return lg;
}

// 2:4 structured sparsity along the input axis: keep the two largest magnitudes of every group of four.
std::tuple<Tensor, Tensor> prune_2_4(const Tensor& w) {
  auto x = w.to(at::kFloat).contiguous();
  TORCH_CHECK(x.size(-1) % 4 == 0, "2:4 pruning needs the last dimension to be a multiple of 4");
  auto out = x.clone();
  auto mask = at::zeros_like(x, at::kBool);
  const int64_t n = x.numel() / 4;
  float* p = out.data_ptr<float>();
  bool* m = mask.data_ptr<bool>();
  for (int64_t g = 0; g < n; ++g) {
    int idx[4] = {0, 1, 2, 3};
    std::sort(idx, idx + 4, [&](int a, int b) { return std::fabs(p[g * 4 + a]) > std::fabs(p[g * 4 + b]) || (std::fabs(p[g * 4 + a]) == std::fabs(p[g * 4 + b]) && a < b); });
    m[g * 4 + idx[0]] = m[g * 4 + idx[1]] = true;
    p[g * 4 + idx[2]] = p[g * 4 + idx[3]] = 0.f;
  }
  return {out.to(w.scalar_type()), mask};
}

}  // namespace

TORCH_LIBRARY_FRAGMENT(mmb200, m) {
  m.def("arena_create", &arena_create);
  m.def("arena_destroy", &arena_destroy);
  m.def("arena_alloc", &arena_alloc);
  m.def("arena_free", &arena_free);
  m.def("arena_pin", &arena_pin);
  m.def("arena_touch", &arena_touch);
  m.def("arena_stats", &arena_stats);
  m.def("arena_compact", &arena_compact);
  m.def("cpu_group_tokens", &cpu_group_tokens);
  m.def("plan_grouped_gemm", &plan_grouped_gemm);
  m.def("cpu_dequant_fp4", &cpu_dequant_fp4);
  m.def("cpu_dequant_codebook", &cpu_dequant_codebook);
  m.def("cpu_router_topk", &cpu_router_topk);
  m.def("cpu_logits_process", &cpu_logits_process);
  m.def("prune_2_4", &prune_2_4);
}

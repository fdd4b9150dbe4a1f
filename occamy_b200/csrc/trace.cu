// Recording, matching and analysis of per-inference call traces (see trace.h).
#include "trace.h"

#include <cstdlib>
#include <cstring>

#include "runtime.h"

namespace occ {

namespace {

struct TraceProgram {
  std::vector<uint64_t> sigs;
  std::vector<uint8_t> roles;
};

struct TraceState {
  int enabled = -1;
  bool in_inference = false;
  bool matched_so_far = false;   // at least one recorded program still matches
  std::vector<Entry> rec;
  std::vector<TraceProgram> programs;
  std::vector<int> cands;
  uintptr_t pool_base = 0;
  size_t pool_bytes = 0;
  int elided = 0;
  int64_t fused_chains = 0;
};

TraceState g_ts;

constexpr size_t MAX_ENTRIES = 50000;
constexpr size_t MAX_PROGRAMS = 16;

inline void mix(uint64_t &h, uint64_t v) {
  for (int i = 0; i < 8; ++i) {
    h = (h ^ (v & 0xFF)) * 1099511628211ull;
    v >>= 8;
  }
}

bool overlaps(uintptr_t a, int64_t abytes, uintptr_t b, int64_t bbytes) {
  return a < b + (uintptr_t)bbytes && b < a + (uintptr_t)abytes;
}

bool is_passive(int sym) {
  return sym == S_MEMOFFSET || sym == S_MALLOC || sym == S_H2D || sym == S_DEALLOC;
}

// True when nothing reads [p, p+bytes) from entry `from` on until the range is handed out
// again, freed, or the inference ends.
bool dies_unread(const std::vector<Entry> &rec, uintptr_t p, int64_t bytes, size_t from) {
  for (size_t t = from; t < rec.size(); ++t) {
    const Entry &e = rec[t];
    for (int k = 0; k < 3; ++k)   // any overlap with an input counts as a read
      if (e.in[k] && overlaps(e.in[k], e.in_bytes[k] > 0 ? e.in_bytes[k] : 1, p, bytes)) return false;
    if ((e.sym == S_MEMOFFSET || e.sym == S_MALLOC) && overlaps(e.out, e.out_bytes, p, bytes))
      return true;
    if ((e.sym == S_DEALLOC && e.out == p) || e.sym == S_POOLFREE) return true;
    if (e.sym == S_OPAQUE) return false;
  }
  return true;
}

bool same_dims(const Entry &a, const Entry &b) {
  return a.dims[0] == b.dims[0] && a.dims[1] == b.dims[1] && a.dims[2] == b.dims[2] &&
         a.dims[3] == b.dims[3];
}

// Marks the chains of a finished inference: R_DEFER on the convolution, R_ABSORB on the
// calls folded into it.
void analyse(const std::vector<Entry> &rec, std::vector<uint8_t> &roles) {
  roles.assign(rec.size(), R_EAGER);
  for (size_t i = 0; i < rec.size(); ++i) {
    const Entry &c = rec[i];
    if ((c.sym != S_CONV && c.sym != S_CONV_BIAS_ACT) || !c.fusable) continue;
    bool bias_set = c.sym == S_CONV_BIAS_ACT;
    bool act_set = c.sym == S_CONV_BIAS_ACT && c.kind != 5;
    bool res_set = false;
    uintptr_t cur = c.out;
    const int64_t cur_bytes = c.out_bytes;
    std::vector<size_t> members;
    for (size_t j = i + 1; j < rec.size() && !act_set; ++j) {
      const Entry &f = rec[j];
      if (is_passive(f.sym)) {
        // the chain's running tensor must stay in place until it is consumed
        if ((f.sym == S_MEMOFFSET || f.sym == S_MALLOC) && overlaps(f.out, f.out_bytes, cur, cur_bytes))
          break;
        if (f.sym == S_DEALLOC && f.out == cur) break;
        continue;
      }
      bool take = false;
      if (f.sym == S_TENSOR_OP && f.kind == CK_BIAS_ADD && f.in[0] == cur && !bias_set && !res_set &&
          same_dims(f, c)) {
        take = true;
      } else if (f.sym == S_TENSOR_OP && f.kind == CK_SAME_ADD && !res_set && !c.depthwise &&
                 ((f.in[0] == cur) != (f.in[1] == cur)) && same_dims(f, c)) {
        take = true;
      } else if ((f.sym == S_ACTIVE && f.kind == CK_RELU) || (f.sym == S_CLIP && f.kind == CK_CLIP)) {
        take = f.in[0] == cur && same_dims(f, c);
      }
      if (!take) break;
      // skipping the write of `cur` is allowed only if this call was its sole reader
      if (f.out != cur && !dies_unread(rec, cur, cur_bytes, j + 1)) break;
      if (f.sym == S_TENSOR_OP && f.kind == CK_BIAS_ADD) bias_set = true;
      else if (f.sym == S_TENSOR_OP) res_set = true;
      else act_set = true;
      members.push_back(j);
      cur = f.out;
    }
    // a stem convolution takes the max pool behind it along, when the pool is the only
    // reader of the full-resolution tensor
    if (c.poolable && !res_set) {
      const size_t from = members.empty() ? i + 1 : members.back() + 1;
      for (size_t j = from; j < rec.size(); ++j) {
        const Entry &f = rec[j];
        if (is_passive(f.sym)) {
          if ((f.sym == S_MEMOFFSET || f.sym == S_MALLOC) && overlaps(f.out, f.out_bytes, cur, cur_bytes))
            break;
          if (f.sym == S_DEALLOC && f.out == cur) break;
          continue;
        }
        if (f.sym == S_MAXPOOL && f.kind == CK_POOL_3S2 && f.in[0] == cur && f.out != cur &&
            dies_unread(rec, cur, cur_bytes, j + 1))
          members.push_back(j);
        break;
      }
    }
    if (members.empty()) continue;
    roles[i] = R_DEFER;
    for (size_t m : members) roles[m] = R_ABSORB;
  }
}

}  // namespace

bool trace_enabled() {
  if (g_ts.enabled < 0) {
    const char *e = getenv("OCCAMY_FUSE_ACROSS_CALLS");
    g_ts.enabled = (e && !strcmp(e, "0")) ? 0 : 1;
  }
  return g_ts.enabled == 1;
}

void trace_set_enabled(bool on) {
  g_ts.enabled = on ? 1 : 0;
  if (!on) {
    g_ts.programs.clear();
    g_ts.cands.clear();
    g_ts.rec.clear();
    g_ts.in_inference = false;
  }
}

Entry trace_entry(int sym) {
  Entry e;
  e.sym = sym;
  mix(e.sig, (uint64_t)sym);
  return e;
}

void te_ptr(Entry &e, const void *p) {
  uintptr_t a = (uintptr_t)p;
  if (g_ts.pool_base && a >= g_ts.pool_base && a < g_ts.pool_base + g_ts.pool_bytes)
    a = (a - g_ts.pool_base) | (1ull << 63);
  mix(e.sig, (uint64_t)a);
}
void te_i(Entry &e, int64_t v) { mix(e.sig, (uint64_t)v); }
void te_f(Entry &e, float v) {
  uint32_t u;
  memcpy(&u, &v, 4);
  mix(e.sig, u);
}
void te_dims(Entry &e, const int64_t *d, int n) {
  for (int i = 0; i < n; ++i) mix(e.sig, (uint64_t)d[i]);
}

Role trace_step(Entry &e, bool *deviated) {
  *deviated = false;
  TraceState &ts = g_ts;
  if (!trace_enabled() || !ts.in_inference) return R_EAGER;
  if (ts.rec.size() >= MAX_ENTRIES) {  // not a compiled model's call pattern: stop tracing
    ts.in_inference = false;
    *deviated = ts.matched_so_far;
    ts.matched_so_far = false;
    return R_EAGER;
  }
  const size_t index = ts.rec.size();
  Role role = R_EAGER;
  if (!ts.cands.empty()) {
    size_t keep = 0;
    for (size_t k = 0; k < ts.cands.size(); ++k) {
      const TraceProgram &p = ts.programs[ts.cands[k]];
      if (index < p.sigs.size() && p.sigs[index] == e.sig) ts.cands[keep++] = ts.cands[k];
    }
    ts.cands.resize(keep);
    if (keep) {
      // recorded programs that share this prefix must agree on the call's role (two models
      // with the same first layers may continue differently); otherwise it runs as it stands
      role = (Role)ts.programs[ts.cands[0]].roles[index];
      for (size_t k = 1; k < keep; ++k)
        if ((Role)ts.programs[ts.cands[k]].roles[index] != role) role = R_EAGER;
      ts.matched_so_far = true;
    } else {
      *deviated = ts.matched_so_far;
      ts.matched_so_far = false;
    }
  }
  ts.rec.push_back(e);
  return role;
}

void trace_begin() {
  TraceState &ts = g_ts;
  if (!trace_enabled()) return;
  ts.in_inference = true;
  ts.matched_so_far = false;
  ts.rec.clear();
  ts.elided = 0;
  ts.cands.clear();
  for (size_t i = 0; i < ts.programs.size(); ++i) ts.cands.push_back((int)i);
}

void trace_end() {
  TraceState &ts = g_ts;
  if (!trace_enabled() || !ts.in_inference) return;
  ts.in_inference = false;
  bool known = false;
  for (int c : ts.cands)
    if (ts.programs[c].sigs.size() == ts.rec.size()) known = true;
  if (!known && !ts.rec.empty()) {
    TraceProgram p;
    p.sigs.reserve(ts.rec.size());
    for (const Entry &e : ts.rec) p.sigs.push_back(e.sig);
    analyse(ts.rec, p.roles);
    if (ts.programs.size() >= MAX_PROGRAMS) ts.programs.erase(ts.programs.begin());
    ts.programs.push_back(std::move(p));
  }
  ts.rec.clear();
  ts.cands.clear();
}

void trace_set_pool(void *base, size_t bytes) {
  g_ts.pool_base = (uintptr_t)base;
  g_ts.pool_bytes = bytes;
}

void trace_note_elided() {
  g_ts.elided++;
}
bool trace_has_elided() { return g_ts.elided > 0; }
int64_t trace_fused_chains() { return g_ts.fused_chains; }
void trace_count_chain() { g_ts.fused_chains++; }

}  // namespace occ

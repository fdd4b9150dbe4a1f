// Host-side stand-in for a model compiled by the Occamy compiler.
//
// The compiler cannot be built without MLIR, so this file restates the part of it that
// fixes WHICH runtime calls a graph turns into and WHERE every tensor lives:
//   * the ONNX->DNN lowering patterns (src/Conversion/ONNXToDNN/Ops/**): Conv ->
//     [malloc workspace][malloc y] convfwd + in-place bias add; Relu -> malloc +
//     activationfwd; Add, MaxPool, AveragePool, ReduceMean (global average pool),
//     Flatten, Gemm (matmul2d + add C), Clip, Softmax; constants -> malloc + H2D copy at
//     first use (ONNXToDNN/Ops/Constant.cpp:85-90); function arguments -> H2D
//     (Transform/DNN/FunctionArgument.cpp:30-53); results -> D2H (ONNXToDNNCommon.cpp:129-183)
//   * the optional conv+bias(+relu) fusion (Transform/DNN/opFusing/fuseConvBiasRelu.cpp:35-154)
//   * dealloc placement right after the last use (Transform/DNN/DNNDeallocOpt.cpp:26-45)
//   * the memory-pool planner: 32-byte rounding, first fit over an address-ordered free
//     list, coalescing free, pool size = high-water mark
//     (Transform/DNN/mallocPoolOpt.hpp:21-140, mallocPoolOpt.cpp:41-76)
// and then replays the resulting straight-line program against any shared library that
// exports the runtime ABI (DNNToLLVM/DNNAPISpecs.inc), exactly as main_graph would.
#include <dlfcn.h>

#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <algorithm>
#include <cstring>
#include <string>
#include <vector>

namespace {

typedef void *Handle;
typedef void *Stream;

struct Api {
  void *so = nullptr;
  int (*cudnnCreate)(Handle *) = nullptr;
  int (*cudnnDestroy)(Handle) = nullptr;
  int (*cudaStreamCreate)(Stream *) = nullptr;
  int (*cudaStreamDestroy)(Stream) = nullptr;
  int (*cudaDeviceSynchronize)() = nullptr;
  int (*wrapDNNMalloc)(void **, size_t) = nullptr;
  int (*wrapDNNMemPoolInit)(void **, size_t) = nullptr;
  int (*wrapDNNMemOffset)(void **, void *, size_t, size_t) = nullptr;
  int (*wrapDNNMemcpy)(void *, const void *, size_t, int, Stream) = nullptr;
  int (*wrapDNNDealloc)(void *) = nullptr;
  float *(*DNNConvFunc)(Handle, float *, int64_t *, float *, int64_t *, float *, int64_t, int64_t,
                        int64_t, int64_t *, int64_t *, float *) = nullptr;
  float *(*DNNConvBiasActivFunc)(Handle, float *, int64_t *, float *, int64_t *, float *,
                                 int64_t *, float *, int64_t, int64_t, int64_t *, int64_t *,
                                 int64_t, float *) = nullptr;
  float *(*DNNActiveFunc)(Handle, float *, int64_t *, int32_t, float *) = nullptr;
  float *(*DNNTensorOpFunc)(Handle, int64_t, float *, int64_t *, int32_t, float *, int64_t *,
                            int32_t, float *, int64_t *, int32_t, float) = nullptr;
  float *(*DNNMaxPoolFunc)(Handle, float *, int64_t *, float *, int64_t *, int64_t *, int64_t *,
                           int64_t *) = nullptr;
  float *(*DNNAveragePoolFunc)(Handle, float *, int64_t *, float *, int64_t *, int64_t *,
                               int64_t *, int64_t *) = nullptr;
  float *(*DNNReduceFunc)(Handle, int32_t, float *, int64_t *, float *, int64_t *, int32_t) = nullptr;
  float *(*CUBLASMatmul2dFunc)(int64_t, float *, int64_t *, float *, int64_t *, float *, int64_t *,
                               float *, int64_t *, float, float, int64_t, int64_t) = nullptr;
  float *(*CUDASoftmaxFunc)(float *, int64_t *, float *, int64_t *, int64_t, int64_t) = nullptr;
  float *(*CUDAClipFunc)(float *, float *, int64_t *, float, float, int64_t) = nullptr;
  float *(*CUDAFlattenFunc)(float *, int64_t *, float *, int64_t *, int32_t, int64_t) = nullptr;
  int (*occamy_synchronize)() = nullptr;  // optional
  std::string error;
};

template <typename F>
bool bind(Api &api, F &fn, const char *name, bool required = true) {
  fn = reinterpret_cast<F>(dlsym(api.so, name));
  if (!fn && required) {
    api.error = std::string("missing symbol ") + name;
    return false;
  }
  return true;
}

enum ValKind { V_INPUT, V_CONST, V_ACT };

struct Value {
  ValKind kind = V_ACT;
  int rank = 0;
  int64_t dims[4] = {1, 1, 1, 1};
  const float *host = nullptr;  // constants: data the "compiled model" embeds
  int buffer = -1;              // device buffer that holds it after lowering
  int64_t numel() const {
    int64_t n = 1;
    for (int i = 0; i < rank; ++i) n *= dims[i];
    return n;
  }
};

enum NodeKind { N_CONV, N_RELU, N_CLIP, N_ADD, N_MAXPOOL, N_AVGPOOL, N_GAP, N_FLATTEN, N_GEMM, N_SOFTMAX };

struct Node {
  NodeKind kind;
  int in[3] = {-1, -1, -1};
  int out = -1;
  int64_t groups = 1, pads[4] = {0, 0, 0, 0}, strides[2] = {1, 1}, kernel[2] = {1, 1};
  float lo = 0.f, hi = 0.f, alpha = 1.f, beta = 1.f;
  int64_t transA = 0, transB = 0, axis = 1;
  bool dead = false;  // absorbed by a fusion
};

// ---- lowered program ----------------------------------------------------------
enum InstrKind {
  I_MALLOC, I_DEALLOC, I_H2D_CONST, I_H2D_INPUT, I_D2H_OUTPUT,
  I_CONV, I_CONV_BIAS_ACT, I_TENSOR_OP, I_ACTIVE, I_CLIP, I_MAXPOOL, I_AVGPOOL, I_REDUCE,
  I_FLATTEN, I_MATMUL, I_SOFTMAX
};

struct Buffer {
  int64_t bytes = 0;       // exact tensor bytes
  int64_t offset = -1;     // pool offset (pool mode)
  void *dev = nullptr;     // run-time address
};

struct Instr {
  InstrKind kind;
  int buf[4] = {-1, -1, -1, -1};   // operand buffers; meaning per kind, output last used slot
  int out = -1;                    // output buffer (also listed for liveness)
  int val = -1;                    // value carrying host data / dims for copies
  int64_t dA[4] = {1, 1, 1, 1}, dB[4] = {1, 1, 1, 1}, dO[4] = {1, 1, 1, 1};
  int rA = 4, rB = 4, rO = 4;
  int64_t pads[4] = {0, 0, 0, 0}, strides[2] = {1, 1}, kernel[2] = {1, 1};
  int64_t groups = 1, mode = 0, ws_bytes = 0, transA = 0, transB = 0, axis = 0;
  float f0 = 0.f, f1 = 0.f;
  int out_index = -1;  // which program output a D2H copy fills
};

struct Program {
  std::vector<Value> vals;
  std::vector<Node> nodes;
  std::vector<int> outputs;
  // lowered
  std::vector<Buffer> bufs;
  std::vector<Instr> prog;
  bool pool = true;
  int pool_mode = 1;       // 1: the reference's first fit; 2: offline greedy-by-size
  int64_t live_peak = 0;   // lower bound of any plan: most bytes live at one time
  int64_t pool_bytes = 0;
  int64_t sum_bytes = 0;   // sum of all buffer sizes (what per-tensor cudaMalloc would total)
  int64_t counts[16] = {0};
  std::string error;
};

int new_val(Program &p, ValKind k, const int64_t *dims, int rank, const float *host) {
  Value v;
  v.kind = k;
  v.rank = rank;
  for (int i = 0; i < rank && i < 4; ++i) v.dims[i] = dims[i];
  v.host = host;
  p.vals.push_back(v);
  return (int)p.vals.size() - 1;
}

int64_t round32(int64_t b) { return b <= 0 ? 0 : ((b - 1) / 32 + 1) * 32; }

// ---- pool planner: first fit over an address-ordered free list -------------------
struct Block {
  int64_t start, end;  // inclusive bounds, as in the reference's simulator
};

struct Planner {
  std::vector<Block> free_list{{0, INT64_MAX - 1}};
  struct Alloc { int buf; int64_t start, end; };
  std::vector<Alloc> allocs;
  int64_t high_water = 0;

  int64_t alloc(int buf, int64_t size) {
    size_t fi = 0;
    for (; fi < free_list.size(); ++fi)
      if (free_list[fi].end - free_list[fi].start >= size) break;
    const int64_t at = free_list[fi].start;
    allocs.push_back(Alloc{buf, at, at + size - 1});
    free_list[fi].start += size;
    if (free_list.back().start > high_water) high_water = free_list.back().start;
    return at;
  }

  void release(int buf) {
    for (size_t ai = 0; ai < allocs.size(); ++ai) {
      if (allocs[ai].buf != buf) continue;
      const Alloc a = allocs[ai];
      allocs.erase(allocs.begin() + ai);
      if (a.end < a.start) return;  // zero-sized
      // merge with a free block that ends right before or starts right after
      for (size_t fi = 0; fi < free_list.size(); ++fi) {
        if (free_list[fi].end == a.start - 1) {
          free_list[fi].end = a.end;
          if (fi + 1 < free_list.size() && free_list[fi + 1].start == free_list[fi].end + 1) {
            free_list[fi + 1].start = free_list[fi].start;
            free_list.erase(free_list.begin() + fi);
          }
          return;
        }
        if (free_list[fi].start == a.end + 1) {
          free_list[fi].start = a.start;
          if (fi > 0 && free_list[fi - 1].end == free_list[fi].start - 1) {
            free_list[fi - 1].end = free_list[fi].end;
            free_list.erase(free_list.begin() + fi);
          }
          return;
        }
      }
      for (size_t fi = 0; fi < free_list.size(); ++fi)
        if (free_list[fi].start > a.end) {
          free_list.insert(free_list.begin() + fi, Block{a.start, a.end});
          return;
        }
      free_list.push_back(Block{a.start, a.end});
      return;
    }
  }
};

// ---- lowering -------------------------------------------------------------------
struct Lowering {
  Program &p;
  int fuse;
  int64_t ws_bytes;
  std::vector<int> uses_left;  // per value: remaining consumer count (for const-at-use)
  explicit Lowering(Program &pp, int f, int64_t ws) : p(pp), fuse(f), ws_bytes(ws) {}

  int new_buf(int64_t bytes) {
    Buffer b;
    b.bytes = bytes;
    p.bufs.push_back(b);
    Instr m;
    m.kind = I_MALLOC;
    m.out = (int)p.bufs.size() - 1;
    p.prog.push_back(m);
    return m.out;
  }

  // device buffer of a value; constants are uploaded right before their first use
  int buf_of(int v) {
    Value &val = p.vals[v];
    if (val.buffer >= 0) return val.buffer;
    if (val.kind == V_CONST) {
      val.buffer = new_buf(val.numel() * 4);
      Instr c;
      c.kind = I_H2D_CONST;
      c.out = val.buffer;
      c.val = v;
      p.prog.push_back(c);
      return val.buffer;
    }
    p.error = "value used before it is defined";
    return 0;
  }

  static void set_dims(int64_t *dst, int *rank, const Value &v) {
    *rank = v.rank;
    for (int i = 0; i < 4; ++i) dst[i] = i < v.rank ? v.dims[i] : 1;
  }

  void run() {
    // function arguments first
    for (size_t v = 0; v < p.vals.size(); ++v)
      if (p.vals[v].kind == V_INPUT) {
        p.vals[v].buffer = new_buf(p.vals[v].numel() * 4);
        Instr c;
        c.kind = I_H2D_INPUT;
        c.out = p.vals[v].buffer;
        c.val = (int)v;
        p.prog.push_back(c);
      }
    // consumers per value, to recognise conv -> add(bias) -> relu/clip chains
    std::vector<std::vector<int>> users(p.vals.size());
    for (size_t n = 0; n < p.nodes.size(); ++n)
      for (int k = 0; k < 3; ++k)
        if (p.nodes[n].in[k] >= 0) users[p.nodes[n].in[k]].push_back((int)n);

    for (size_t ni = 0; ni < p.nodes.size(); ++ni) {
      Node &nd = p.nodes[ni];
      if (nd.dead) continue;
      const Value &x = p.vals[nd.in[0]];
      Value &y = p.vals[nd.out];
      Instr in;
      switch (nd.kind) {
        case N_CONV: {
          const int xb = buf_of(nd.in[0]);
          const int wb = buf_of(nd.in[1]);
          const int wsb = new_buf(ws_bytes);
          // Fusion: the only consumer of the conv result is a Relu (reference pass) or,
          // with fuse == 2, a Clip(0, 6).  The bias add is part of the Conv pattern.
          int act_mode = -1, act_node = -1;
          const bool has_bias = nd.in[2] >= 0;
          if (fuse && has_bias && nd.groups == 1) {
            act_mode = 5;
            if (users[nd.out].size() == 1) {
              Node &u = p.nodes[users[nd.out][0]];
              if (u.kind == N_RELU) { act_mode = 1; act_node = users[nd.out][0]; }
              else if (fuse == 2 && u.kind == N_CLIP && u.lo == 0.f && u.hi == 6.f) {
                act_mode = 3; act_node = users[nd.out][0];
              }
            }
          }
          in.groups = nd.groups;
          in.pads[0] = nd.pads[0]; in.pads[1] = nd.pads[1];
          in.strides[0] = nd.strides[0]; in.strides[1] = nd.strides[1];
          in.ws_bytes = ws_bytes;
          set_dims(in.dA, &in.rA, x);
          set_dims(in.dB, &in.rB, p.vals[nd.in[1]]);
          if (act_mode >= 0) {
            const int bb = buf_of(nd.in[2]);
            int target = nd.out;
            if (act_node >= 0) {
              target = p.nodes[act_node].out;
              p.nodes[act_node].dead = true;
            }
            const int yb = new_buf(p.vals[target].numel() * 4);
            p.vals[target].buffer = yb;
            y.buffer = yb;
            in.kind = I_CONV_BIAS_ACT;
            in.buf[0] = xb; in.buf[1] = wb; in.buf[2] = bb; in.buf[3] = wsb;
            in.out = yb;
            in.mode = act_mode;
            in.dO[0] = 1; in.dO[1] = y.dims[1]; in.dO[2] = 1; in.dO[3] = 1;  // bias dims
            p.prog.push_back(in);
          } else {
            const int yb = new_buf(y.numel() * 4);
            y.buffer = yb;
            in.kind = I_CONV;
            in.buf[0] = xb; in.buf[1] = wb; in.buf[3] = wsb;
            in.out = yb;
            p.prog.push_back(in);
            if (has_bias) {
              Instr add;
              add.kind = I_TENSOR_OP;
              add.mode = 0;
              add.buf[0] = yb; add.buf[1] = buf_of(nd.in[2]);
              add.out = yb;
              set_dims(add.dA, &add.rA, y);
              add.rB = 4; add.dB[0] = 1; add.dB[1] = y.dims[1]; add.dB[2] = 1; add.dB[3] = 1;
              set_dims(add.dO, &add.rO, y);
              add.f0 = 1.f;
              p.prog.push_back(add);
            }
          }
          break;
        }
        case N_RELU:
        case N_CLIP: {
          const int xb = buf_of(nd.in[0]);
          y.buffer = new_buf(y.numel() * 4);
          in.kind = nd.kind == N_RELU ? I_ACTIVE : I_CLIP;
          in.buf[0] = xb; in.out = y.buffer;
          in.mode = 1; in.f0 = nd.lo; in.f1 = nd.hi;
          set_dims(in.dA, &in.rA, x);
          p.prog.push_back(in);
          break;
        }
        case N_ADD: {
          const int ab = buf_of(nd.in[0]), bb = buf_of(nd.in[1]);
          y.buffer = new_buf(y.numel() * 4);
          in.kind = I_TENSOR_OP;
          in.mode = 0; in.f0 = 1.f;
          in.buf[0] = ab; in.buf[1] = bb; in.out = y.buffer;
          set_dims(in.dA, &in.rA, x);
          set_dims(in.dB, &in.rB, p.vals[nd.in[1]]);
          set_dims(in.dO, &in.rO, y);
          p.prog.push_back(in);
          break;
        }
        case N_MAXPOOL:
        case N_AVGPOOL: {
          const int xb = buf_of(nd.in[0]);
          y.buffer = new_buf(y.numel() * 4);
          in.kind = nd.kind == N_MAXPOOL ? I_MAXPOOL : I_AVGPOOL;
          in.buf[0] = xb; in.out = y.buffer;
          set_dims(in.dA, &in.rA, x);
          set_dims(in.dO, &in.rO, y);
          for (int i = 0; i < 4; ++i) in.pads[i] = nd.pads[i];
          for (int i = 0; i < 2; ++i) { in.kernel[i] = nd.kernel[i]; in.strides[i] = nd.strides[i]; }
          p.prog.push_back(in);
          break;
        }
        case N_GAP: {
          const int xb = buf_of(nd.in[0]);
          y.buffer = new_buf(y.numel() * 4);
          in.kind = I_REDUCE;
          in.mode = 5;
          in.buf[0] = xb; in.out = y.buffer;
          set_dims(in.dA, &in.rA, x);
          set_dims(in.dO, &in.rO, y);
          p.prog.push_back(in);
          break;
        }
        case N_FLATTEN: {
          const int xb = buf_of(nd.in[0]);
          y.buffer = new_buf(y.numel() * 4);
          in.kind = I_FLATTEN;
          in.axis = 1;
          in.buf[0] = xb; in.out = y.buffer;
          set_dims(in.dA, &in.rA, x);
          set_dims(in.dO, &in.rO, y);
          p.prog.push_back(in);
          break;
        }
        case N_GEMM: {
          const int ab = buf_of(nd.in[0]), bb = buf_of(nd.in[1]);
          y.buffer = new_buf(y.numel() * 4);
          in.kind = I_MATMUL;
          in.buf[0] = ab; in.buf[1] = bb; in.out = y.buffer;
          set_dims(in.dA, &in.rA, x);
          set_dims(in.dB, &in.rB, p.vals[nd.in[1]]);
          set_dims(in.dO, &in.rO, y);
          in.f0 = nd.alpha; in.f1 = nd.beta;
          in.transA = nd.transA; in.transB = nd.transB;
          p.prog.push_back(in);
          if (nd.in[2] >= 0) {
            Instr add;
            add.kind = I_TENSOR_OP;
            add.mode = 0; add.f0 = 1.f;
            add.buf[0] = y.buffer; add.buf[1] = buf_of(nd.in[2]); add.out = y.buffer;
            set_dims(add.dA, &add.rA, y);
            add.rB = 2; add.dB[0] = 1; add.dB[1] = y.dims[1];
            set_dims(add.dO, &add.rO, y);
            p.prog.push_back(add);
          }
          break;
        }
        case N_SOFTMAX: {
          const int xb = buf_of(nd.in[0]);
          y.buffer = new_buf(y.numel() * 4);
          in.kind = I_SOFTMAX;
          in.axis = nd.axis;
          in.buf[0] = xb; in.out = y.buffer;
          set_dims(in.dA, &in.rA, x);
          set_dims(in.dO, &in.rO, y);
          p.prog.push_back(in);
          break;
        }
      }
    }
    for (size_t oi = 0; oi < p.outputs.size(); ++oi) {
      Instr c;
      c.kind = I_D2H_OUTPUT;
      c.buf[0] = buf_of(p.outputs[oi]);
      c.val = p.outputs[oi];
      c.out_index = (int)oi;
      p.prog.push_back(c);
    }
  }
};

// Put one dealloc per buffer: right after its last use (dealloc_opt) or at the end.
void place_deallocs(Program &p, bool dealloc_opt) {
  const int nb = (int)p.bufs.size();
  std::vector<int> last(nb, -1);
  for (size_t i = 0; i < p.prog.size(); ++i) {
    const Instr &in = p.prog[i];
    for (int k = 0; k < 4; ++k)
      if (in.buf[k] >= 0) last[in.buf[k]] = (int)i;
    if (in.out >= 0) last[in.out] = (int)i;
  }
  std::vector<Instr> out;
  out.reserve(p.prog.size() + nb);
  std::vector<std::vector<int>> dying(p.prog.size());
  for (int b = 0; b < nb; ++b) {
    const int at = dealloc_opt ? last[b] : (int)p.prog.size() - 1;
    dying[at].push_back(b);
  }
  for (size_t i = 0; i < p.prog.size(); ++i) {
    out.push_back(p.prog[i]);
    for (int b : dying[i]) {
      Instr d;
      d.kind = I_DEALLOC;
      d.out = b;
      out.push_back(d);
    }
  }
  p.prog.swap(out);
}

// Most bytes live at any point of the program: no plan can use less.
static int64_t live_bytes_peak(const Program &p) {
  int64_t live = 0, peak = 0;
  for (const Instr &in : p.prog) {
    if (in.kind == I_MALLOC) live += round32(p.bufs[in.out].bytes);
    else if (in.kind == I_DEALLOC) live -= round32(p.bufs[in.out].bytes);
    if (live > peak) peak = live;
  }
  return peak;
}

// Offline plan (not the reference's): a compiled model is straight-line code, so every
// buffer's lifetime [malloc, dealloc] is known before anything is placed.  Buffers go in
// order of decreasing size, each at the lowest offset where it overlaps no already placed
// buffer that is live at the same time.  The online first fit below has to place buffers in
// program order and fragments around long-lived ones.
static void plan_pool_by_size(Program &p) {
  struct Item { int buf; int64_t size; int from, to; int64_t offset; };
  std::vector<Item> items;
  std::vector<int> item_of(p.bufs.size(), -1);
  for (size_t i = 0; i < p.prog.size(); ++i) {
    const Instr &in = p.prog[i];
    if (in.kind == I_MALLOC) {
      item_of[in.out] = (int)items.size();
      items.push_back(Item{in.out, round32(p.bufs[in.out].bytes), (int)i, (int)p.prog.size(), 0});
    } else if (in.kind == I_DEALLOC && item_of[in.out] >= 0) {
      items[item_of[in.out]].to = (int)i;
    }
  }
  std::vector<int> order(items.size());
  for (size_t i = 0; i < order.size(); ++i) order[i] = (int)i;
  std::stable_sort(order.begin(), order.end(),
                   [&](int a, int b) { return items[a].size > items[b].size; });
  std::vector<int> placed;
  int64_t high = 0;
  for (int idx : order) {
    Item &it = items[idx];
    // offsets of the placed buffers that are live together with this one, in address order
    std::vector<std::pair<int64_t, int64_t>> busy;
    for (int q : placed) {
      const Item &o = items[q];
      if (o.from <= it.to && it.from <= o.to && o.size > 0) busy.push_back({o.offset, o.offset + o.size});
    }
    std::sort(busy.begin(), busy.end());
    int64_t at = 0;
    for (const auto &b : busy) {
      if (b.first - at >= it.size) break;
      if (b.second > at) at = b.second;
    }
    it.offset = at;
    p.bufs[it.buf].offset = at;
    if (at + it.size > high) high = at + it.size;
    placed.push_back(idx);
  }
  p.pool_bytes = high;
}

void plan_pool(Program &p) {
  Planner pl;
  p.sum_bytes = 0;
  for (const Instr &in : p.prog) {
    if (in.kind == I_MALLOC) {
      const int64_t sz = round32(p.bufs[in.out].bytes);
      p.bufs[in.out].offset = pl.alloc(in.out, sz);
      p.sum_bytes += sz;
    } else if (in.kind == I_DEALLOC) {
      pl.release(in.out);
    }
  }
  p.pool_bytes = pl.high_water;
  p.live_peak = live_bytes_peak(p);
  if (p.pool_mode == 2) plan_pool_by_size(p);
}

}  // namespace

// ================================ C API =========================================
extern "C" {

void *occ_prog_create() { return new Program(); }
void occ_prog_destroy(void *h) { delete static_cast<Program *>(h); }
const char *occ_prog_error(void *h) { return static_cast<Program *>(h)->error.c_str(); }

int occ_v_input(void *h, const int64_t *dims, int rank) {
  return new_val(*static_cast<Program *>(h), V_INPUT, dims, rank, nullptr);
}
int occ_v_const(void *h, const float *host, const int64_t *dims, int rank) {
  return new_val(*static_cast<Program *>(h), V_CONST, dims, rank, host);
}
void occ_mark_output(void *h, int v) { static_cast<Program *>(h)->outputs.push_back(v); }

void occ_v_dims(void *h, int v, int64_t *dims, int *rank) {
  const Value &val = static_cast<Program *>(h)->vals[v];
  *rank = val.rank;
  for (int i = 0; i < 4; ++i) dims[i] = val.dims[i];
}

static int add_node(Program &p, Node nd, const int64_t *odims, int orank) {
  nd.out = new_val(p, V_ACT, odims, orank, nullptr);
  p.nodes.push_back(nd);
  return nd.out;
}

int occ_op_conv(void *h, int x, int w, int b, int groups, int pad_h, int pad_w, int stride_h,
                int stride_w) {
  Program &p = *static_cast<Program *>(h);
  const Value &X = p.vals[x], &W = p.vals[w];
  Node nd;
  nd.kind = N_CONV;
  nd.in[0] = x; nd.in[1] = w; nd.in[2] = b;
  nd.groups = groups;
  nd.pads[0] = pad_h; nd.pads[1] = pad_w;
  nd.strides[0] = stride_h; nd.strides[1] = stride_w;
  const int64_t od[4] = {X.dims[0], W.dims[0], (X.dims[2] + 2 * pad_h - W.dims[2]) / stride_h + 1,
                         (X.dims[3] + 2 * pad_w - W.dims[3]) / stride_w + 1};
  return add_node(p, nd, od, 4);
}

static int unary_node(Program &p, NodeKind k, int x, float lo, float hi) {
  Node nd;
  nd.kind = k;
  nd.in[0] = x;
  nd.lo = lo; nd.hi = hi;
  return add_node(p, nd, p.vals[x].dims, p.vals[x].rank);
}
int occ_op_relu(void *h, int x) { return unary_node(*static_cast<Program *>(h), N_RELU, x, 0, 0); }
int occ_op_clip(void *h, int x, float lo, float hi) {
  return unary_node(*static_cast<Program *>(h), N_CLIP, x, lo, hi);
}
int occ_op_add(void *h, int a, int b) {
  Program &p = *static_cast<Program *>(h);
  Node nd;
  nd.kind = N_ADD;
  nd.in[0] = a; nd.in[1] = b;
  return add_node(p, nd, p.vals[a].dims, p.vals[a].rank);
}

static int pool_node(Program &p, NodeKind k, int x, int kh, int kw, int pad_h, int pad_w, int sh,
                     int sw) {
  const Value &X = p.vals[x];
  Node nd;
  nd.kind = k;
  nd.in[0] = x;
  nd.kernel[0] = kh; nd.kernel[1] = kw;
  // ONNX attribute order (h_begin, w_begin, h_end, w_end), passed through unchanged by the
  // lowering (ONNXToDNN/Ops/cudnn/MaxPoolSingleOut.cpp:56-63); the runtime takes the
  // vertical pad from [0] and the horizontal one from [2], so only square padding is exact.
  nd.pads[0] = pad_h; nd.pads[1] = pad_w; nd.pads[2] = pad_h; nd.pads[3] = pad_w;
  nd.strides[0] = sh; nd.strides[1] = sw;
  const int64_t od[4] = {X.dims[0], X.dims[1], (X.dims[2] + 2 * pad_h - kh) / sh + 1,
                         (X.dims[3] + 2 * pad_w - kw) / sw + 1};
  return add_node(p, nd, od, 4);
}
int occ_op_maxpool(void *h, int x, int kh, int kw, int pad_h, int pad_w, int sh, int sw) {
  return pool_node(*static_cast<Program *>(h), N_MAXPOOL, x, kh, kw, pad_h, pad_w, sh, sw);
}
int occ_op_avgpool(void *h, int x, int kh, int kw, int pad_h, int pad_w, int sh, int sw) {
  return pool_node(*static_cast<Program *>(h), N_AVGPOOL, x, kh, kw, pad_h, pad_w, sh, sw);
}
int occ_op_gap(void *h, int x) {
  Program &p = *static_cast<Program *>(h);
  Node nd;
  nd.kind = N_GAP;
  nd.in[0] = x;
  const int64_t od[4] = {p.vals[x].dims[0], p.vals[x].dims[1], 1, 1};
  return add_node(p, nd, od, 4);
}
int occ_op_flatten(void *h, int x) {
  Program &p = *static_cast<Program *>(h);
  Node nd;
  nd.kind = N_FLATTEN;
  nd.in[0] = x;
  const Value &X = p.vals[x];
  const int64_t od[4] = {X.dims[0], X.numel() / X.dims[0], 1, 1};
  return add_node(p, nd, od, 2);
}
int occ_op_gemm(void *h, int a, int b, int c, float alpha, float beta, int transA, int transB) {
  Program &p = *static_cast<Program *>(h);
  Node nd;
  nd.kind = N_GEMM;
  nd.in[0] = a; nd.in[1] = b; nd.in[2] = c;
  nd.alpha = alpha; nd.beta = beta; nd.transA = transA; nd.transB = transB;
  const Value &A = p.vals[a], &B = p.vals[b];
  const int64_t od[4] = {transA ? A.dims[1] : A.dims[0], transB ? B.dims[0] : B.dims[1], 1, 1};
  return add_node(p, nd, od, 2);
}
int occ_op_softmax(void *h, int x, int axis) {
  Program &p = *static_cast<Program *>(h);
  Node nd;
  nd.kind = N_SOFTMAX;
  nd.in[0] = x;
  nd.axis = axis;
  return add_node(p, nd, p.vals[x].dims, p.vals[x].rank);
}

// fuse: 0 = none (what the reference's test scripts compile), 1 = the reference's
// conv+bias(+relu) fusion, 2 = additionally conv+bias+clip(0,6) -> activMode 3.
// pool_opt: 0 = one wrapDNNMalloc per tensor, 1 = the reference's first-fit pool plan,
// 2 = pool with the offline greedy-by-size plan.
int occ_lower(void *h, int fuse, int dealloc_opt, int pool_opt, int64_t workspace_bytes) {
  Program &p = *static_cast<Program *>(h);
  p.bufs.clear();
  p.prog.clear();
  for (Value &v : p.vals) v.buffer = -1;
  for (Node &n : p.nodes) n.dead = false;
  Lowering lw(p, fuse, workspace_bytes);
  lw.run();
  if (!p.error.empty()) return -1;
  place_deallocs(p, dealloc_opt != 0);
  p.pool = pool_opt != 0;
  p.pool_mode = pool_opt == 2 ? 2 : 1;
  plan_pool(p);
  memset(p.counts, 0, sizeof(p.counts));
  for (const Instr &in : p.prog) p.counts[in.kind]++;
  return (int)p.prog.size();
}

int64_t occ_pool_bytes(void *h) { return static_cast<Program *>(h)->pool_bytes; }
int64_t occ_sum_bytes(void *h) { return static_cast<Program *>(h)->sum_bytes; }
int64_t occ_live_peak_bytes(void *h) { return static_cast<Program *>(h)->live_peak; }
void occ_instr_counts(void *h, int64_t *out16) {
  memcpy(out16, static_cast<Program *>(h)->counts, sizeof(int64_t) * 16);
}
// Planned (offset, bytes) of every buffer, in allocation order; returns the count.
int occ_plan(void *h, int64_t *offsets, int64_t *bytes, int cap) {
  Program &p = *static_cast<Program *>(h);
  int n = 0;
  for (const Instr &in : p.prog)
    if (in.kind == I_MALLOC) {
      if (n < cap) {
        offsets[n] = p.bufs[in.out].offset;
        bytes[n] = round32(p.bufs[in.out].bytes);
      }
      ++n;
    }
  return n;
}

// Lifetime [malloc index, dealloc index] (program positions) of every buffer, in allocation
// order like occ_plan; a buffer that is never freed lives to the end of the program.
int occ_lifetimes(void *h, int64_t *from, int64_t *to, int cap) {
  Program &p = *static_cast<Program *>(h);
  std::vector<int> slot(p.bufs.size(), -1);
  int n = 0;
  for (size_t i = 0; i < p.prog.size(); ++i) {
    const Instr &in = p.prog[i];
    if (in.kind == I_MALLOC) {
      slot[in.out] = n;
      if (n < cap) {
        from[n] = (int64_t)i;
        to[n] = (int64_t)p.prog.size();
      }
      ++n;
    } else if (in.kind == I_DEALLOC && slot[in.out] >= 0 && slot[in.out] < cap) {
      to[slot[in.out]] = (int64_t)i;
    }
  }
  return n;
}

void *occ_bind(const char *so_path, char *err, int err_cap) {
  Api *api = new Api();
  api->so = dlopen(so_path, RTLD_NOW | RTLD_LOCAL);
  bool ok = api->so != nullptr;
  if (!ok) api->error = std::string("dlopen failed: ") + dlerror();
  ok = ok && bind(*api, api->cudnnCreate, "cudnnCreate") && bind(*api, api->cudnnDestroy, "cudnnDestroy") &&
       bind(*api, api->cudaStreamCreate, "cudaStreamCreate") &&
       bind(*api, api->cudaStreamDestroy, "cudaStreamDestroy") &&
       bind(*api, api->cudaDeviceSynchronize, "cudaDeviceSynchronize") &&
       bind(*api, api->wrapDNNMalloc, "wrapDNNMalloc") &&
       bind(*api, api->wrapDNNMemPoolInit, "wrapDNNMemPoolInit") &&
       bind(*api, api->wrapDNNMemOffset, "wrapDNNMemOffset") &&
       bind(*api, api->wrapDNNMemcpy, "wrapDNNMemcpy") && bind(*api, api->wrapDNNDealloc, "wrapDNNDealloc") &&
       bind(*api, api->DNNConvFunc, "DNNConvFunc") &&
       bind(*api, api->DNNConvBiasActivFunc, "DNNConvBiasActivFunc") &&
       bind(*api, api->DNNActiveFunc, "DNNActiveFunc") && bind(*api, api->DNNTensorOpFunc, "DNNTensorOpFunc") &&
       bind(*api, api->DNNMaxPoolFunc, "DNNMaxPoolFunc") &&
       bind(*api, api->DNNAveragePoolFunc, "DNNAveragePoolFunc") &&
       bind(*api, api->DNNReduceFunc, "DNNReduceFunc") &&
       bind(*api, api->CUBLASMatmul2dFunc, "CUBLASMatmul2dFunc") &&
       bind(*api, api->CUDASoftmaxFunc, "CUDASoftmaxFunc") && bind(*api, api->CUDAClipFunc, "CUDAClipFunc") &&
       bind(*api, api->CUDAFlattenFunc, "CUDAFlattenFunc");
  if (ok) bind(*api, api->occamy_synchronize, "occamy_synchronize", false);
  if (!ok) {
    if (err && err_cap > 0) snprintf(err, err_cap, "%s", api->error.c_str());
    delete api;
    return nullptr;
  }
  return api;
}

// One inference: replays the lowered program.  `input_kind` 1: `input` is host memory
// (H2D copy, as the compiled model does); 3: `input` is device memory (device-to-device
// copy; used to time the path with the batch already resident).  `outputs[i]` receives
// program output i through the D2H copy (copy_out 1).  copy_out 0: no output copy, the
// function waits for the device instead.  copy_out 3: `outputs[i]` are device buffers
// filled by device-to-device copies and the function returns without waiting (the caller
// orders its own work on the runtime's stream).  Returns 0, or a negative code.
int occ_run(void *h, void *api_h, const float *input, int input_kind, float **outputs,
            int copy_out) {
  Program &p = *static_cast<Program *>(h);
  Api &api = *static_cast<Api *>(api_h);
  Handle handle = nullptr;
  Stream stream = nullptr;
  api.cudnnCreate(&handle);
  api.cudaStreamCreate(&stream);
  void *pool = nullptr;
  if (p.pool) api.wrapDNNMemPoolInit(&pool, (size_t)p.pool_bytes);
  for (Instr &in : p.prog) {
    float *b0 = in.buf[0] >= 0 ? (float *)p.bufs[in.buf[0]].dev : nullptr;
    float *b1 = in.buf[1] >= 0 ? (float *)p.bufs[in.buf[1]].dev : nullptr;
    float *b2 = in.buf[2] >= 0 ? (float *)p.bufs[in.buf[2]].dev : nullptr;
    float *b3 = in.buf[3] >= 0 ? (float *)p.bufs[in.buf[3]].dev : nullptr;
    float *o = in.out >= 0 ? (float *)p.bufs[in.out].dev : nullptr;
    switch (in.kind) {
      case I_MALLOC: {
        Buffer &b = p.bufs[in.out];
        if (p.pool) api.wrapDNNMemOffset(&b.dev, pool, (size_t)b.offset, (size_t)round32(b.bytes));
        else api.wrapDNNMalloc(&b.dev, (size_t)b.bytes);
        break;
      }
      case I_DEALLOC:
        if (!p.pool) api.wrapDNNDealloc(p.bufs[in.out].dev);
        break;
      case I_H2D_CONST:
        api.wrapDNNMemcpy(o, p.vals[in.val].host, (size_t)p.bufs[in.out].bytes, 1, stream);
        break;
      case I_H2D_INPUT:
        api.wrapDNNMemcpy(o, input, (size_t)p.bufs[in.out].bytes, input_kind, stream);
        break;
      case I_D2H_OUTPUT:
        // copy_out 1: device->host as the compiled model does; 3: device->device into a
        // caller-owned device buffer (the result stays on the GPU for a collective)
        if (copy_out)
          api.wrapDNNMemcpy(outputs[in.out_index], b0, (size_t)p.vals[in.val].numel() * 4,
                            copy_out == 3 ? 3 : 2, stream);
        break;
      case I_CONV:
        // algorithm 0 (implicit GEMM) needs no workspace, whatever size the plan reserved; the
        // real compiler passes whichever algorithm cuDNN's search picked on its machine
        api.DNNConvFunc(handle, b0, in.dA, b1, in.dB, b3, in.ws_bytes, 0, in.groups, in.pads,
                        in.strides, o);
        break;
      case I_CONV_BIAS_ACT:
        api.DNNConvBiasActivFunc(handle, b0, in.dA, b1, in.dB, b2, in.dO, b3, in.ws_bytes, 1,
                                 in.pads, in.strides, in.mode, o);
        break;
      case I_TENSOR_OP:
        api.DNNTensorOpFunc(handle, in.mode, b0, in.dA, in.rA, b1, in.dB, in.rB, o, in.dO, in.rO,
                            in.f0);
        break;
      case I_ACTIVE:
        api.DNNActiveFunc(handle, b0, in.dA, (int32_t)in.mode, o);
        break;
      case I_CLIP:
        api.CUDAClipFunc(b0, o, in.dA, in.f0, in.f1, in.rA);
        break;
      case I_MAXPOOL:
        api.DNNMaxPoolFunc(handle, b0, in.dA, o, in.dO, in.kernel, in.pads, in.strides);
        break;
      case I_AVGPOOL:
        api.DNNAveragePoolFunc(handle, b0, in.dA, o, in.dO, in.kernel, in.pads, in.strides);
        break;
      case I_REDUCE:
        api.DNNReduceFunc(handle, in.rA, b0, in.dA, o, in.dO, (int32_t)in.mode);
        break;
      case I_FLATTEN:
        api.CUDAFlattenFunc(b0, in.dA, o, in.dO, (int32_t)in.axis, in.rA);
        break;
      case I_MATMUL:
        api.CUBLASMatmul2dFunc(2, b0, in.dA, b1, in.dB, o, in.dO, o, in.dO, in.f0, in.f1, in.transA,
                               in.transB);
        break;
      case I_SOFTMAX:
        api.CUDASoftmaxFunc(b0, in.dA, o, in.dO, in.axis, in.rA);
        break;
    }
  }
  if (copy_out == 0) {
    if (api.occamy_synchronize) api.occamy_synchronize();
    else api.cudaDeviceSynchronize();
  }
  if (p.pool) api.wrapDNNDealloc(pool);
  else api.cudaDeviceSynchronize();
  api.cudaStreamDestroy(stream);
  api.cudnnDestroy(handle);
  return 0;
}

}  // extern "C"

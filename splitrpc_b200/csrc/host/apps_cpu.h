// CPU implementations of the apps: the oracle for the GPU kernels and the apps of
// the GPU-less plumbing configuration.
//
// Every app is the usual four callbacks {init, run, cleanup, complete} over an
// AppCtx; per-instance state hangs off app_ctx->app_ctx_internal.  A run reads
// curr_batch_size requests starting at h_stub->req and writes as many responses
// starting at h_stub->resp (the ring window is contiguous).
//   echo     resp = req                               (reference src/apps/echo_rpc_bench.cc:25-36)
//   vec_add  resp[i] = req[i] + 1 (uint8)             (reference src/apps/vec_add/vector_add.cu:22-35)
//   matmul   C = A.B, fp32 square, A and B packed     (reference src/apps/mm.cu:12-36)
//   lenet5   conv5x5(1->6,pad 2)-relu-maxpool-conv5x5(6->16)-relu-maxpool-
//            fc120-relu-fc84-relu-fc10-softmax, fp32; request 1x28x28 fp32,
//            response 10 fp32 probabilities
//   lenet_ref  the 20/50/10 network of reference src/apps/lenet/lenet_vanilla.cu:17-192
//            (uint8 pixels, (x-127)/128, conv pad 1, tanh, maxpool, dense, softmax)
#pragma once

#include <atomic>
#include <cmath>
#include <condition_variable>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <functional>
#include <memory>
#include <mutex>
#include <sstream>
#include <string>
#include <thread>
#include <vector>

#include "cpu_batch_pool.h"
#include "p2p_rpc_app.h"

struct CpuAppState {
  size_t req_size = 0, resp_size = 0;
  std::vector<std::vector<float>> weights;  // app specific
  int dim = 0;                              // matmul dimension
  std::unique_ptr<CpuBatchPool> pool;       // created by the first batch that can use it
  // Requests of one batch spread over the caller and up to three helper threads (P2P_RPC_CPU_APP_THREADS, default
  // min(4, half of the cores)).
  CpuBatchPool* batch_pool() {
    if (!pool) {
      int want = 0;
      if (const char* e = getenv("P2P_RPC_CPU_APP_THREADS")) want = atoi(e);
      if (want <= 0) {
        const int hw = (int)std::thread::hardware_concurrency();
        want = hw / 2 < 4 ? (hw / 2 > 1 ? hw / 2 : 1) : 4;
      }
      pool.reset(new CpuBatchPool(want - 1));
    }
    return pool.get();
  }
};

static inline CpuAppState* cpu_state(AppCtx* c) { return static_cast<CpuAppState*>(c->app_ctx_internal); }

static inline int cpu_app_noop(AppCtx*) { return 1; }

// ---- echo
static inline int cpu_echo_run(AppCtx* c) {
  CpuAppState* s = cpu_state(c);
  size_t copy = s->req_size < s->resp_size ? s->req_size : s->resp_size;
  for (int b = 0; b < c->curr_batch_size; b++)
    std::memcpy(c->h_stub->resp + (size_t)b * s->resp_size, c->h_stub->req + (size_t)b * s->req_size, copy);
  return 1;
}

// ---- vec_add
static inline int cpu_vec_add_run(AppCtx* c) {
  CpuAppState* s = cpu_state(c);
  size_t n = (s->req_size < s->resp_size ? s->req_size : s->resp_size);
  for (int b = 0; b < c->curr_batch_size; b++) {
    const uint8_t* in = c->h_stub->req + (size_t)b * s->req_size;
    uint8_t* out = c->h_stub->resp + (size_t)b * s->resp_size;
    for (size_t i = 0; i < n; i++) out[i] = (uint8_t)(in[i] + 1);
  }
  return 1;
}

// ---- matmul: request = A (d*d fp32) followed by B (d*d fp32); response = C
static inline int mm_dim_from_req(size_t req_size) {
  int d = (int)std::lround(std::sqrt((double)req_size / 8.0));
  return d;
}
static inline int cpu_mm_run(AppCtx* c) {
  CpuAppState* s = cpu_state(c);
  const int d = s->dim ? s->dim : mm_dim_from_req(s->req_size);
  const uint8_t* req = c->h_stub->req;
  uint8_t* resp = c->h_stub->resp;
  s->batch_pool()->run(c->curr_batch_size, [s, d, req, resp](int b) {
    const float* A = reinterpret_cast<const float*>(req + (size_t)b * s->req_size);
    const float* B = A + (size_t)d * d;
    float* C = reinterpret_cast<float*>(resp + (size_t)b * s->resp_size);
    // row of C += A[i][k] * row k of B: the inner loop runs along contiguous memory
    for (int i = 0; i < d; i++) {
      float* ci = C + (size_t)i * d;
      for (int j = 0; j < d; j++) ci[j] = 0.f;
      for (int k = 0; k < d; k++) {
        const float a = A[(size_t)i * d + k];
        const float* bk = B + (size_t)k * d;
        for (int j = 0; j < d; j++) ci[j] += a * bk[j];
      }
    }
  });
  return 1;
}

// ---- generic layers (NCHW, fp32)
static inline void cpu_conv2d(const float* in, int C, int H, int W, const float* w, const float* bias, int K, int R,
                              int pad, float* out) {
  // One filter tap at a time over whole output rows: the inner loop is a contiguous multiply-add (vectorised by the
  // compiler), and the padding turns into loop bounds instead of a test per element.
  const int OH = H + 2 * pad - R + 1, OW = W + 2 * pad - R + 1;
  for (int k = 0; k < K; k++) {
    float* ok = out + (size_t)k * OH * OW;
    const float b = bias ? bias[k] : 0.f;
    for (int i = 0; i < OH * OW; i++) ok[i] = b;
    for (int c = 0; c < C; c++)
      for (int r = 0; r < R; r++) {
        const int oh_lo = pad - r > 0 ? pad - r : 0, oh_hi = H + pad - r < OH ? H + pad - r : OH;
        for (int q = 0; q < R; q++) {
          const int ow_lo = pad - q > 0 ? pad - q : 0, ow_hi = W + pad - q < OW ? W + pad - q : OW;
          const float wv = w[((k * C + c) * R + r) * R + q];
          for (int oh = oh_lo; oh < oh_hi; oh++) {
            float* o = ok + oh * OW;
            const float* x = in + (c * H + oh + r - pad) * W + (q - pad);
            for (int ow = ow_lo; ow < ow_hi; ow++) o[ow] += x[ow] * wv;
          }
        }
      }
  }
}
static inline void cpu_maxpool2(const float* in, int C, int H, int W, float* out) {
  int OH = H / 2, OW = W / 2;
  for (int c = 0; c < C; c++)
    for (int oh = 0; oh < OH; oh++)
      for (int ow = 0; ow < OW; ow++) {
        const float* p = in + (c * H + 2 * oh) * W + 2 * ow;
        out[(c * OH + oh) * OW + ow] = std::fmax(std::fmax(p[0], p[1]), std::fmax(p[W], p[W + 1]));
      }
}
static inline void cpu_dense(const float* in, int n_in, const float* w, const float* bias, int n_out, float* out) {
  for (int o = 0; o < n_out; o++) {
    // eight partial sums: a plain running sum is a dependency chain that the compiler may not reorder
    float part[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const float* wr = w + (size_t)o * n_in;
    int i = 0;
    for (; i + 8 <= n_in; i += 8)
      for (int j = 0; j < 8; j++) part[j] += in[i + j] * wr[i + j];
    float acc = bias ? bias[o] : 0.f;
    for (; i < n_in; i++) acc += in[i] * wr[i];
    out[o] = acc + ((part[0] + part[1]) + (part[2] + part[3])) + ((part[4] + part[5]) + (part[6] + part[7]));
  }
}
static inline void cpu_softmax(float* v, int n) {
  float m = v[0];
  for (int i = 1; i < n; i++) m = std::fmax(m, v[i]);
  float s = 0.f;
  for (int i = 0; i < n; i++) {
    v[i] = std::exp(v[i] - m);
    s += v[i];
  }
  for (int i = 0; i < n; i++) v[i] /= s;
}

// ---- LeNet-5.  weights: 0 conv1 W[6,1,5,5] 1 conv1 b[6] 2 conv2 W[16,6,5,5] 3 conv2 b[16]
//      4 fc1 W[120,400] 5 fc1 b 6 fc2 W[84,120] 7 fc2 b 8 fc3 W[10,84] 9 fc3 b
static constexpr size_t LENET5_REQ_BYTES = 28 * 28 * 4;
static constexpr size_t LENET5_RESP_BYTES = 10 * 4;
static inline void cpu_lenet5_one(const CpuAppState* s, const float* x, float* y) {
  float a1[6 * 28 * 28], p1[6 * 14 * 14], a2[16 * 10 * 10], p2[16 * 5 * 5], f1[120], f2[84];
  const auto& w = s->weights;
  cpu_conv2d(x, 1, 28, 28, w[0].data(), w[1].data(), 6, 5, 2, a1);
  for (float& v : a1) v = v > 0.f ? v : 0.f;
  cpu_maxpool2(a1, 6, 28, 28, p1);
  cpu_conv2d(p1, 6, 14, 14, w[2].data(), w[3].data(), 16, 5, 0, a2);
  for (float& v : a2) v = v > 0.f ? v : 0.f;
  cpu_maxpool2(a2, 16, 10, 10, p2);
  cpu_dense(p2, 400, w[4].data(), w[5].data(), 120, f1);
  for (float& v : f1) v = v > 0.f ? v : 0.f;
  cpu_dense(f1, 120, w[6].data(), w[7].data(), 84, f2);
  for (float& v : f2) v = v > 0.f ? v : 0.f;
  cpu_dense(f2, 84, w[8].data(), w[9].data(), 10, y);
  cpu_softmax(y, 10);
}
static inline int cpu_lenet5_run(AppCtx* c) {
  CpuAppState* s = cpu_state(c);
  const uint8_t* req = c->h_stub->req;
  uint8_t* resp = c->h_stub->resp;
  s->batch_pool()->run(c->curr_batch_size, [s, req, resp](int b) {
    cpu_lenet5_one(s, reinterpret_cast<const float*>(req + (size_t)b * s->req_size),
                   reinterpret_cast<float*>(resp + (size_t)b * s->resp_size));
  });
  return 1;
}

// ---- reference-format LeNet.  weights: 0 conv1 W[20,1,5,5] 1 conv2 W[50,20,5,5] 2 fc W[10,1250] 3 fc b[10]
static inline void cpu_lenet_ref_one(const CpuAppState* s, const uint8_t* px, float* y) {
  std::vector<float> x(784), a1(20 * 26 * 26), p1(20 * 13 * 13), a2(50 * 11 * 11), p2(50 * 5 * 5);
  const auto& w = s->weights;
  for (int i = 0; i < 784; i++) x[i] = ((float)px[i] - 127.f) / 128.f;
  cpu_conv2d(x.data(), 1, 28, 28, w[0].data(), nullptr, 20, 5, 1, a1.data());
  for (float& v : a1) v = std::tanh(v);
  cpu_maxpool2(a1.data(), 20, 26, 26, p1.data());
  cpu_conv2d(p1.data(), 20, 13, 13, w[1].data(), nullptr, 50, 5, 1, a2.data());
  for (float& v : a2) v = std::tanh(v);
  cpu_maxpool2(a2.data(), 50, 11, 11, p2.data());
  cpu_dense(p2.data(), 1250, w[2].data(), w[3].data(), 10, y);
  cpu_softmax(y, 10);
}
static inline int cpu_lenet_ref_run(AppCtx* c) {
  CpuAppState* s = cpu_state(c);
  const uint8_t* req = c->h_stub->req;
  uint8_t* resp = c->h_stub->resp;
  s->batch_pool()->run(c->curr_batch_size, [s, req, resp](int b) {
    cpu_lenet_ref_one(s, req + (size_t)b * s->req_size, reinterpret_cast<float*>(resp + (size_t)b * s->resp_size));
  });
  return 1;
}

// Reads the four raw little-endian fp32 blobs of the reference LeNet format from
// <dir>/data/lenet/{data2,data0,data1,data3}.dat (conv1 W, conv2 W, fc W, fc b;
// reference src/apps/lenet/lenet_vanilla.cu:445-484).
static inline bool load_lenet_ref_weights(const std::string& dataset_dir, std::vector<std::vector<float>>* out) {
  static const char* files[4] = {"data2.dat", "data0.dat", "data1.dat", "data3.dat"};
  static const size_t counts[4] = {500, 25000, 12500, 10};
  out->assign(4, {});
  for (int i = 0; i < 4; i++) {
    std::ifstream f(dataset_dir + "/data/lenet/" + files[i], std::ios::binary);
    if (!f) return false;
    (*out)[i].resize(counts[i]);
    f.read(reinterpret_cast<char*>((*out)[i].data()), (std::streamsize)(counts[i] * 4));
    if ((size_t)f.gcount() != counts[i] * 4) return false;
  }
  return true;
}

// Reads the LSTM's weights from the original's per-constant files: <dir>/Constant_<id>_0.bin, raw fp32, one file per
// tensor (64 matrices of H x H, 32 vectors of H for the 8-layer model; reference
// src/apps/nnfusion_lstm/nnfusion_rt.cu:13884-13896 and the Constant/ directory beside it).  Which constant is which
// tensor is a property of the exported graph, not of the file format, so it comes from a manifest: one line per tensor,
//     <layer> <W|U|b> <gate: i|g|f|o> <constant id> [T]
// W multiplies the layer's input, U its previous hidden state; T marks a matrix stored [in][out] (the layout a
// Dot(x, M) node consumes), which is transposed into the [out][in] rows used here.  Lines starting with # are
// comments.  Output: per layer W[4][H][H], U[4][H][H], b[4][H] in gate order i, g, f, o (what the apps take).
// Returns an empty string on success, else what went wrong.
static inline std::string load_lstm_constant_dir(const std::string& dir, const std::string& manifest_path, int layers, int H,
                                                 std::vector<std::vector<float>>* out) {
  std::ifstream mf(manifest_path);
  if (!mf) return "cannot open manifest " + manifest_path;
  out->assign((size_t)3 * layers, {});
  for (int l = 0; l < layers; l++) {
    (*out)[3 * l].assign((size_t)4 * H * H, 0.f);
    (*out)[3 * l + 1].assign((size_t)4 * H * H, 0.f);
    (*out)[3 * l + 2].assign((size_t)4 * H, 0.f);
  }
  std::vector<uint8_t> seen((size_t)layers * 12, 0);
  float forget_bias = 0.f;
  std::string line;
  int line_no = 0;
  std::vector<float> buf;
  while (std::getline(mf, line)) {
    line_no++;
    if (line.empty() || line[0] == '#') continue;
    std::istringstream ss(line);
    if (line.compare(0, 11, "forget_bias") == 0) {  // "forget_bias <value>": added to every forget-gate bias
      std::string word;
      if (!(ss >> word >> forget_bias)) return "manifest line " + std::to_string(line_no) + ": expected forget_bias <value>";
      continue;
    }
    int layer = -1, id = -1;
    std::string kind, gate, flag;
    if (!(ss >> layer >> kind >> gate >> id)) return "manifest line " + std::to_string(line_no) + ": expected <layer> <W|U|b> <gate> <id>";
    ss >> flag;
    const int k = kind == "W" ? 0 : (kind == "U" ? 1 : (kind == "b" ? 2 : -1));
    const int g = gate == "i" ? 0 : (gate == "g" ? 1 : (gate == "f" ? 2 : (gate == "o" ? 3 : -1)));
    if (layer < 0 || layer >= layers || k < 0 || g < 0 || id < 0) return "manifest line " + std::to_string(line_no) + ": bad field";
    const size_t count = k == 2 ? (size_t)H : (size_t)H * H;
    const std::string path = dir + "/Constant_" + std::to_string(id) + "_0.bin";
    std::ifstream f(path, std::ios::binary);
    if (!f) return "missing " + path;
    buf.resize(count);
    f.read(reinterpret_cast<char*>(buf.data()), (std::streamsize)(count * 4));
    if ((size_t)f.gcount() != count * 4) return path + " is shorter than " + std::to_string(count * 4) + " bytes";
    float* dst = (*out)[3 * layer + k].data() + (size_t)g * count;
    if (k < 2 && flag == "T") {
      for (int o = 0; o < H; o++)
        for (int i = 0; i < H; i++) dst[(size_t)o * H + i] = buf[(size_t)i * H + o];
    } else {
      std::memcpy(dst, buf.data(), count * 4);
    }
    seen[(size_t)layer * 12 + (size_t)k * 4 + g] = 1;
  }
  for (size_t i = 0; i < seen.size(); i++)
    if (!seen[i]) return "manifest does not name layer " + std::to_string(i / 12) + " tensor " + std::to_string((i % 12) / 4) + " gate " + std::to_string(i % 4);
  if (forget_bias != 0.f)  // the cell of the apps adds no constant of its own: fold it into the bias (gate order i, g, f, o)
    for (int l = 0; l < layers; l++)
      for (int j = 0; j < H; j++) (*out)[3 * l + 2][(size_t)2 * H + j] += forget_bias;
  return "";
}

// ---- LSTM cell math of the stacked 8-layer x 8-step, hidden 256 model
// (reference src/apps/nnfusion_lstm/nnfusion_rt.cu:1213-1283): gates from
// W.x + U.h + b, c' = sigmoid(f + forget_bias)*c + sigmoid(i)*tanh(g),
// h' = tanh(c') * sigmoid(o).  weights per layer: W[4][H][H], U[4][H][H], b[4][H]
// in gate order i, g(cell), f, o.  Request {steps, 1, H} fp32, response {1, H}.
static inline float cpu_sigmoid(float x) { return 1.f / (1.f + std::exp(-x)); }
static inline void cpu_lstm_forward(const std::vector<std::vector<float>>& w, int layers, int steps, int H,
                                    float forget_bias, const float* x, float* y) {
  std::vector<float> seq(x, x + (size_t)steps * H), next((size_t)steps * H);
  std::vector<float> h(H), cst(H), gates(4 * (size_t)H);
  for (int l = 0; l < layers; l++) {
    const float* W = w[3 * l].data();
    const float* U = w[3 * l + 1].data();
    const float* b = w[3 * l + 2].data();
    std::fill(h.begin(), h.end(), 0.f);
    std::fill(cst.begin(), cst.end(), 0.f);
    for (int t = 0; t < steps; t++) {
      const float* xt = seq.data() + (size_t)t * H;
      for (int g = 0; g < 4; g++)
        for (int o = 0; o < H; o++) {
          float acc = b[g * H + o];
          const float* wr = W + ((size_t)g * H + o) * H;
          const float* ur = U + ((size_t)g * H + o) * H;
          for (int k = 0; k < H; k++) acc += wr[k] * xt[k] + ur[k] * h[k];
          gates[(size_t)g * H + o] = acc;
        }
      for (int o = 0; o < H; o++) {
        float ig = gates[o], gg = gates[H + o], fg = gates[2 * H + o], og = gates[3 * H + o];
        cst[o] = cpu_sigmoid(fg + forget_bias) * cst[o] + cpu_sigmoid(ig) * std::tanh(gg);
        h[o] = std::tanh(cst[o]) * cpu_sigmoid(og);
        next[(size_t)t * H + o] = h[o];
      }
    }
    seq.swap(next);
  }
  std::memcpy(y, seq.data() + (size_t)(steps - 1) * H, (size_t)H * 4);
}
static inline int cpu_lstm_run(AppCtx* c) {
  CpuAppState* s = cpu_state(c);
  const int H = 256, steps = 8, layers = 8;
  const uint8_t* req = c->h_stub->req;
  uint8_t* resp = c->h_stub->resp;
  s->batch_pool()->run(c->curr_batch_size, [s, req, resp](int b) {
    cpu_lstm_forward(s->weights, layers, steps, H, 0.0f, reinterpret_cast<const float*>(req + (size_t)b * s->req_size),
                     reinterpret_cast<float*>(resp + (size_t)b * s->resp_size));
  });
  return 1;
}

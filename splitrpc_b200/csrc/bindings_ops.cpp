// Python bindings of the CUDA kernels.  Tensors cross this boundary as raw device
// addresses (int) plus shapes; the Python layer owns allocation through PyTorch.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cuda_runtime.h>

#include "cuda/gemm_tcgen05.h"
#include "cuda/gemm_tp.h"
#include "cuda/nn_kernels.h"
#include "cuda/ops_api.h"
#include "host/p2p_rpc.h"
#include "host/p2p_rpc_app.h"
#include "cuda/parity_kernels.h"

namespace py = pybind11;

static void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

static GemmEpilogue make_ep(uintptr_t out, int ldo, bool out_fp32, uintptr_t bias, uintptr_t residual, int ldr, int act) {
  GemmEpilogue ep;
  ep.out = (void*)out;
  ep.ldo = ldo;
  ep.out_fp32 = out_fp32 ? 1 : 0;
  ep.bias = (const float*)bias;
  ep.residual = (const __nv_bfloat16*)residual;
  ep.ldr = ldr;
  ep.act = act;
  return ep;
}

extern "C" int srpc_stream_write64(cudaStream_t s, uint64_t* addr, uint64_t v);
extern "C" int srpc_stream_wait32_geq(cudaStream_t s, uint32_t* addr, uint32_t v);

void bind_ops(py::module_& m) {
  m.def("device_caps", [](int dev) {
    int vmm = 0, memops = 0, gdr = 0, maj = 0, min = 0, nsm = 0;
    py::dict d;
    if (srpc_device_caps(dev, &vmm, &memops, &gdr, &maj, &min, &nsm) != 0) return d;
    d["vmm"] = vmm;
    d["stream_memops"] = memops;
    d["gdr_with_vmm"] = gdr;
    d["sm"] = maj * 10 + min;
    d["num_sms"] = nsm;
    return d;
  });

  // ---- scatter-gather
  m.def("sg_copy",
        [](const std::vector<SgTuple>& items, int impl, int n_blocks, uintptr_t stream) {
          check(srpc_sg_copy_list(items, impl, n_blocks, (cudaStream_t)stream), "sg_copy");
        },
        py::arg("items"), py::arg("impl") = 0, py::arg("n_blocks") = 0, py::arg("stream") = 0);
  m.def("sg_cast_bf16",
        [](const std::vector<SgTuple>& items, float scale, float shift, int n_blocks, uintptr_t stream) {
          check(srpc_sg_cast_list(items, scale, shift, n_blocks, (cudaStream_t)stream), "sg_cast_bf16");
        },
        py::arg("items"), py::arg("scale") = 1.0f, py::arg("shift") = 0.0f, py::arg("n_blocks") = 0, py::arg("stream") = 0);
  m.def("memset_async", [](uintptr_t dst, int value, size_t n, uintptr_t stream) {
    check(cudaMemsetAsync((void*)dst, value, n, (cudaStream_t)stream), "memset_async");
  });
  m.def("memcpy2d_async", [](uintptr_t dst, size_t dpitch, uintptr_t src, size_t spitch, size_t width, size_t height,
                             uintptr_t stream) {
    check(cudaMemcpy2DAsync((void*)dst, dpitch, (const void*)src, spitch, width, height, cudaMemcpyDefault, (cudaStream_t)stream),
          "memcpy2d_async");
  });
  m.def("memcpy_async", [](uintptr_t dst, uintptr_t src, size_t n, uintptr_t stream) {
    check(cudaMemcpyAsync((void*)dst, (const void*)src, n, cudaMemcpyDefault, (cudaStream_t)stream), "memcpy_async");
  });
  m.def("sg_list_create", &srpc_sg_list_create, py::arg("items"), py::arg("bells") = std::vector<uint64_t>{});
  m.def("sg_list_destroy", &srpc_sg_list_destroy);
  m.def("sg_list_launch_stem_s2d",
        [](uintptr_t h, uintptr_t ring_base, uint32_t slot_bytes, std::vector<float> mean, std::vector<float> inv_std, int n_blocks,
           uintptr_t stream, uint32_t bell_value, uintptr_t done_word, uint32_t done_value) {
          if (mean.size() != 3 || inv_std.size() != 3) throw std::invalid_argument("mean / inv_std need 3 values");
          check(srpc_sg_list_launch_stem_s2d(h, ring_base, slot_bytes, mean.data(), inv_std.data(), n_blocks, (cudaStream_t)stream,
                                             bell_value, done_word, done_value),
                "sg_list_launch_stem_s2d");
        },
        py::arg("handle"), py::arg("ring_base"), py::arg("slot_bytes"), py::arg("mean"), py::arg("inv_std"), py::arg("n_blocks") = 0,
        py::arg("stream") = 0, py::arg("bell_value") = 0, py::arg("done_word") = 0, py::arg("done_value") = 0);
  m.def("sg_list_launch",
        [](uintptr_t h, int impl, int n_blocks, uintptr_t stream, uint32_t bell_value, uintptr_t done_word, uint32_t done_value) {
          check(srpc_sg_list_launch(h, impl, n_blocks, (cudaStream_t)stream, bell_value, done_word, done_value), "sg_list_launch");
        },
        py::arg("handle"), py::arg("impl") = 0, py::arg("n_blocks") = 0, py::arg("stream") = 0, py::arg("bell_value") = 0,
        py::arg("done_word") = 0, py::arg("done_value") = 0);
  // Stream-ordered doorbell operations on a 32-bit word that the device can address (mapped host memory or device
  // memory): the stream waits until the word equals `value` / writes `value` once everything queued before has finished.
  m.def("stream_wait32", [](uintptr_t stream, uintptr_t addr, uint32_t value, bool geq) {
    const SrpcDeviceOps* o = srpc_cuda_ops();
    // geq: the word is a sequence number that only grows; wait until it has reached `value` (cyclic comparison)
    int rc = !o ? -1 : (geq ? srpc_stream_wait32_geq((cudaStream_t)stream, (uint32_t*)addr, value)
                            : o->stream_wait_value32((cudaStream_t)stream, (volatile uint32_t*)addr, value));
    if (rc != 0) throw std::runtime_error(std::string("stream_wait32: ") + (o ? o->last_error() : "no CUDA"));
  }, py::arg("stream"), py::arg("addr"), py::arg("value"), py::arg("geq") = false);
  m.def("stream_write64", [](uintptr_t stream, uintptr_t addr, uint64_t value) {
    const SrpcDeviceOps* o = srpc_cuda_ops();
    if (!o || srpc_stream_write64((cudaStream_t)stream, (uint64_t*)addr, value) != 0)
      throw std::runtime_error(std::string("stream_write64: ") + (o ? o->last_error() : "no CUDA"));
  });
  m.def("stream_write32", [](uintptr_t stream, uintptr_t addr, uint32_t value) {
    const SrpcDeviceOps* o = srpc_cuda_ops();
    if (!o || o->stream_write_value32((cudaStream_t)stream, (volatile uint32_t*)addr, value) != 0)
      throw std::runtime_error(std::string("stream_write32: ") + (o ? o->last_error() : "no CUDA"));
  });

  // ---- tensor-core GEMM / convolution
  m.attr("ACT_NONE") = (int)GEMM_ACT_NONE;
  m.attr("ACT_RELU") = (int)GEMM_ACT_RELU;
  m.attr("ACT_GELU") = (int)GEMM_ACT_GELU;
  m.attr("ACT_TANH") = (int)GEMM_ACT_TANH;
  m.def("gemm_bf16",
        [](uintptr_t a, int lda, uintptr_t b, int ldb, int M, int N, int K, uintptr_t out, int ldo, bool out_fp32,
           uintptr_t bias, uintptr_t residual, int ldr, int act, uintptr_t status, uintptr_t stream, int impl) {
          GemmEpilogue ep = make_ep(out, ldo, out_fp32, bias, residual, ldr, act);
          auto fn = impl == 1 ? srpc_gemm_bf16 : srpc_gemm_bf16_v2;
          check(fn((const void*)a, lda, (const void*)b, ldb, M, N, K, ep, (uint32_t*)status, (cudaStream_t)stream),
                "gemm_bf16");
        },
        py::arg("a"), py::arg("lda"), py::arg("b"), py::arg("ldb"), py::arg("M"), py::arg("N"), py::arg("K"), py::arg("out"),
        py::arg("ldo"), py::arg("out_fp32") = false, py::arg("bias") = 0, py::arg("residual") = 0, py::arg("ldr") = 0,
        py::arg("act") = 0, py::arg("status") = 0, py::arg("stream") = 0, py::arg("impl") = 2);
  m.def("conv_bf16",
        [](uintptr_t in, uintptr_t w, int n, int h, int wd, int cin, int cout, int r, int s, int stride, int pad,
           uintptr_t out, uintptr_t bias, uintptr_t residual, int act, uintptr_t status, uintptr_t stream, int impl,
           long pix_stride, long row_stride, long img_stride, uintptr_t in_stub, long ring_slots, unsigned int slot_bytes,
           uintptr_t in2, int h2, int w2, int cin2, int stride2) {
          ConvShape cs{n, h, wd, cin, cout, r, s, stride, pad, (h + 2 * pad - r) / stride + 1, (wd + 2 * pad - s) / stride + 1};
          cs.in_pix_stride = pix_stride;
          cs.in_row_stride = row_stride;
          cs.in_img_stride = img_stride;
          cs.in_stub = (const void*)in_stub;
          cs.in_ring_slots = ring_slots;
          cs.in_slot_bytes = slot_bytes;
          cs.in2 = (const void*)in2;
          cs.h2 = h2;
          cs.w2 = w2;
          cs.cin2 = cin2;
          cs.stride2 = stride2;
          if (in2 && impl == 1) throw std::invalid_argument("conv_bf16: a second input needs the TMA implementation");
          if ((pix_stride || row_stride || img_stride) && impl == 1)
            throw std::invalid_argument("conv_bf16: input strides need the TMA implementation");
          GemmEpilogue ep = make_ep(out, cout, false, bias, residual, cout, act);
          auto fn = impl == 1 ? srpc_conv_bf16 : srpc_conv_bf16_tma;
          check(fn((const void*)in, (const void*)w, cs, ep, (uint32_t*)status, (cudaStream_t)stream), "conv_bf16");
        },
        py::arg("input"), py::arg("weight"), py::arg("n"), py::arg("h"), py::arg("w"), py::arg("cin"), py::arg("cout"),
        py::arg("r"), py::arg("s"), py::arg("stride"), py::arg("pad"), py::arg("out"), py::arg("bias") = 0,
        py::arg("residual") = 0, py::arg("act") = 0, py::arg("status") = 0, py::arg("stream") = 0, py::arg("impl") = 2,
        py::arg("pix_stride") = 0, py::arg("row_stride") = 0, py::arg("img_stride") = 0, py::arg("in_stub") = 0,
        py::arg("ring_slots") = 0, py::arg("slot_bytes") = 0, py::arg("in2") = 0, py::arg("h2") = 0, py::arg("w2") = 0,
        py::arg("cin2") = 0, py::arg("stride2") = 1);

  m.def("gemm_reserve_sms", [](int n) { srpc_gemm_reserve_sms(n); }, py::arg("n"));
  m.def("gemm_grid_sms", []() { return srpc_gemm_grid_sms(); });
  m.def("gemm_reserved_sms", []() { return srpc_gemm_reserved_sms(); });
  m.def("gemm_trace", [](bool two_sm) {
    unsigned long long t[16] = {0};
    int n = two_sm ? srpc_gemm2_trace_read(t, 12) : srpc_gemm_trace_read(t, 16);
    std::vector<uint64_t> v(t, t + n);
    return v;
  }, py::arg("two_sm") = false);

  // ---- tensor-parallel fused kernels
  m.def("gemm_tp",
        [](uintptr_t a, int lda, uintptr_t b, int ldb, int M, int N, int K, uintptr_t out, int ldo, uintptr_t bias, int act,
           int tp, int rank, uint32_t epoch, uintptr_t mblock_ready, int n_copy, std::vector<uintptr_t> src,
           uintptr_t gathered, uintptr_t src_ready, int rs, std::vector<uintptr_t> dst, std::vector<uintptr_t> dst_flag,
           uintptr_t owner_count, uintptr_t status, uintptr_t stream, uintptr_t epoch_base) {
          GemmEpilogue ep = make_ep(out, ldo, false, bias, 0, 0, act);
          TpParams t;
          t.tp = tp;
          t.rank = rank;
          t.epoch = epoch;
          t.epoch_base = (const uint32_t*)epoch_base;
          t.mblock_ready = (uint32_t*)mblock_ready;
          t.n_copy = n_copy;
          for (size_t i = 0; i < src.size() && i < TP_MAX_RANKS; i++) t.src[i] = (const uint8_t*)src[i];
          t.gathered = (uint8_t*)gathered;
          t.src_ready = (const uint32_t*)src_ready;
          t.rs = rs;
          for (size_t i = 0; i < dst.size() && i < TP_MAX_RANKS; i++) t.dst[i] = (uint8_t*)dst[i];
          for (size_t i = 0; i < dst_flag.size() && i < TP_MAX_RANKS; i++) t.dst_flag[i] = (uint32_t*)dst_flag[i];
          t.owner_count = (uint32_t*)owner_count;
          check(srpc_gemm_tp((const void*)a, lda, (const void*)b, ldb, M, N, K, ep, t, (uint32_t*)status, (cudaStream_t)stream),
                "gemm_tp");
        },
        py::arg("a"), py::arg("lda"), py::arg("b"), py::arg("ldb"), py::arg("M"), py::arg("N"), py::arg("K"), py::arg("out"),
        py::arg("ldo"), py::arg("bias") = 0, py::arg("act") = 0, py::arg("tp") = 1, py::arg("rank") = 0, py::arg("epoch") = 0,
        py::arg("mblock_ready") = 0, py::arg("n_copy") = 0, py::arg("src") = std::vector<uintptr_t>{},
        py::arg("gathered") = 0, py::arg("src_ready") = 0, py::arg("rs") = 0, py::arg("dst") = std::vector<uintptr_t>{},
        py::arg("dst_flag") = std::vector<uintptr_t>{}, py::arg("owner_count") = 0, py::arg("status") = 0,
        py::arg("stream") = 0, py::arg("epoch_base") = 0);
  m.def("tp_set_wait_ns", [](uint64_t ns) { check(srpc_tp_set_wait_ns(ns), "tp_set_wait_ns"); });
  m.def("tp_wait", [](uintptr_t flags, int n, uint32_t epoch, uintptr_t epoch_base, uintptr_t status, uintptr_t stream) {
    check(srpc_tp_wait((const uint32_t*)flags, n, epoch, (const uint32_t*)epoch_base, (uint32_t*)status, (cudaStream_t)stream),
          "tp_wait");
  });
  m.def("tp_begin", [](uintptr_t flags, int n, uintptr_t epoch_base, uint32_t delta, uintptr_t status, uintptr_t stream) {
    check(srpc_tp_begin((const uint32_t*)flags, n, (uint32_t*)epoch_base, delta, (uint32_t*)status, (cudaStream_t)stream),
          "tp_begin");
  });
  m.def("tp_fanout",
        [](uintptr_t d_stub, uint32_t req_bytes, uint32_t batch, uint32_t max_batch, uint32_t command, std::vector<uintptr_t> dst,
           std::vector<uintptr_t> ctrl, std::vector<uintptr_t> doorbell, uintptr_t seq, uintptr_t arrivals, uintptr_t stream) {
          TpFanout f{};
          f.tp = (int)dst.size();
          if (f.tp > TP_MAX_RANKS || ctrl.size() != dst.size() || doorbell.size() != dst.size())
            throw std::invalid_argument("tp_fanout: one destination, control record and doorbell per rank");
          f.stub = (const void*)d_stub;
          f.req_bytes = req_bytes;
          f.batch = batch;
          f.max_batch = max_batch;
          f.command = command;
          for (int r = 0; r < f.tp; r++) {
            f.dst[r] = (uint8_t*)dst[(size_t)r];
            f.ctrl[r] = (uint32_t*)ctrl[(size_t)r];
            f.doorbell[r] = (uint32_t*)doorbell[(size_t)r];
          }
          f.seq = (uint32_t*)seq;
          f.arrivals = (uint32_t*)arrivals;
          check(srpc_tp_fanout(f, (cudaStream_t)stream), "tp_fanout");
        },
        py::arg("d_stub"), py::arg("req_bytes"), py::arg("batch"), py::arg("max_batch"), py::arg("command"), py::arg("dst"),
        py::arg("ctrl"), py::arg("doorbell"), py::arg("seq"), py::arg("arrivals"), py::arg("stream"));
  m.def("tp_bump", [](uintptr_t word, uint32_t delta, uintptr_t stream) {
    check(srpc_tp_bump((uint32_t*)word, delta, (cudaStream_t)stream), "tp_bump");
  });
  m.def("tp_signal", [](std::vector<uintptr_t> peer_flags, uint32_t epoch, uintptr_t stream, uintptr_t epoch_base) {
    TpSignal s{};
    s.tp = (int)peer_flags.size();
    s.epoch = epoch;
    s.epoch_base = (const uint32_t*)epoch_base;
    for (size_t i = 0; i < peer_flags.size() && i < TP_MAX_RANKS; i++) s.peer_flag[i] = (uint32_t*)peer_flags[i];
    check(srpc_tp_signal(s, (cudaStream_t)stream), "tp_signal");
  });
  m.def("layernorm_reduce",
        [](std::vector<uintptr_t> slots, uintptr_t flags, uint32_t epoch, uintptr_t bias, uintptr_t residual, uintptr_t gamma,
           uintptr_t beta, uintptr_t out, int rows, int hidden, float eps, uintptr_t status, uintptr_t stream,
           uintptr_t epoch_base, std::vector<uintptr_t> sig_flags, uint32_t sig_epoch, uintptr_t done_count) {
          TpReduce r{};
          r.tp = (int)slots.size();
          r.hidden = hidden;
          r.epoch = epoch;
          r.epoch_base = (const uint32_t*)epoch_base;
          r.flags = (const uint32_t*)flags;
          for (size_t i = 0; i < slots.size() && i < TP_MAX_RANKS; i++) r.slots[i] = (const __nv_bfloat16*)slots[i];
          r.bias = (const float*)bias;
          r.residual = (const __nv_bfloat16*)residual;
          r.gamma = (const float*)gamma;
          r.beta = (const float*)beta;
          r.out = (__nv_bfloat16*)out;
          r.eps = eps;
          r.sig_tp = done_count ? (int)std::min(sig_flags.size(), (size_t)TP_MAX_RANKS) : 0;
          r.sig_epoch = sig_epoch;
          for (int i = 0; i < r.sig_tp; i++) r.sig_peer_flag[i] = (uint32_t*)sig_flags[i];
          r.done_count = (uint32_t*)done_count;
          check(srpc_layernorm_reduce(r, rows, (uint32_t*)status, (cudaStream_t)stream), "layernorm_reduce");
        },
        py::arg("slots"), py::arg("flags"), py::arg("epoch"), py::arg("bias"), py::arg("residual"), py::arg("gamma"),
        py::arg("beta"), py::arg("out"), py::arg("rows"), py::arg("hidden"), py::arg("eps"), py::arg("status"),
        py::arg("stream"), py::arg("epoch_base"), py::arg("sig_flags") = std::vector<uintptr_t>{}, py::arg("sig_epoch") = 0,
        py::arg("done_count") = 0);

  // GPU header processor: handle = g_pp_setup(device, launch_type); g_pp_do(handle, [addresses], clear_sockperf);
  // g_pp_stop(handle).
  m.def("g_pp_setup", [](int device, int launch_type) {
    pp_handler_ctx* c = setup_g_pp(device, launch_type);
    if (!c) throw std::runtime_error("setup_g_pp failed");
    return (uintptr_t)c;
  }, py::arg("device") = 0, py::arg("launch_type") = -1);
  m.def("g_pp_do", [](uintptr_t h, const std::vector<uint64_t>& hdr_addrs, bool clear_sockperf) {
    auto bufs = std::make_unique<p2p_hbufs>();
    if (hdr_addrs.size() > MAX_BI_SIZE) throw std::invalid_argument("at most 1024 headers per burst");
    bufs->num_items = (uint16_t)hdr_addrs.size();
    for (size_t i = 0; i < hdr_addrs.size(); i++) bufs->burst_items[i] = hdr_addrs[i];
    py::gil_scoped_release rel;
    return do_g_pp((pp_handler_ctx*)h, bufs.get(), clear_sockperf ? 1 : 0);
  }, py::arg("handle"), py::arg("hdr_addrs"), py::arg("clear_sockperf") = false);
  m.def("g_pp_counters", [](uintptr_t h) {
    uint64_t b, r, t;
    int lt;
    g_pp_counters((pp_handler_ctx*)h, &b, &r, &t, &lt);
    py::dict d;
    d["bursts"] = b;
    d["rearmed"] = r;
    d["timeouts"] = t;
    d["launch_type"] = lt;
    return d;
  });
  m.def("g_pp_stop", [](uintptr_t h) { stop_g_pp((pp_handler_ctx*)h); });
  m.def("swap_hdrs", [](uintptr_t hdr_ptrs, uintptr_t hdrs_contig, int n, bool clear_sockperf, uintptr_t stream) {
    check(srpc_swap_hdrs((void* const*)hdr_ptrs, (void*)hdrs_contig, n, clear_sockperf ? 1 : 0, (cudaStream_t)stream), "swap_hdrs");
  });

  // ---- memory-bound layers
  m.def("stem_im2col",
        [](uintptr_t d_stub, uintptr_t direct_in, int batch, uintptr_t out, std::vector<float> mean, std::vector<float> inv_std,
           uintptr_t stream) {
          if (mean.size() != 3 || inv_std.size() != 3) throw std::invalid_argument("mean / inv_std need 3 values");
          check(nn_stem_im2col((const void*)d_stub, (const float*)direct_in, batch, (void*)out, mean.data(), inv_std.data(),
                               (cudaStream_t)stream),
                "stem_im2col");
        });
  m.def("stem_s2d",
        [](uintptr_t d_stub, uintptr_t direct_in, int batch, uintptr_t out, std::vector<float> mean, std::vector<float> inv_std,
           uintptr_t stream) {
          if (mean.size() != 3 || inv_std.size() != 3) throw std::invalid_argument("mean / inv_std need 3 values");
          check(nn_stem_s2d((const void*)d_stub, (const float*)direct_in, batch, (void*)out, mean.data(), inv_std.data(),
                            (cudaStream_t)stream),
                "stem_s2d");
        });
  m.def("maxpool3x3s2", [](uintptr_t in, uintptr_t out, int n, int h, int w, int c, uintptr_t stream) {
    check(nn_maxpool3x3s2((const void*)in, (void*)out, n, h, w, c, (cudaStream_t)stream), "maxpool3x3s2");
  });
  m.def("global_avgpool", [](uintptr_t in, uintptr_t out, int n, int hw, int c, uintptr_t stream) {
    check(nn_global_avgpool((const void*)in, (void*)out, n, hw, c, (cudaStream_t)stream), "global_avgpool");
  });
  m.def("fc_skinny", [](uintptr_t a, int lda, uintptr_t w, int ldw, uintptr_t bias, uintptr_t out, int ldo, int M, int N, int K,
                        uintptr_t stream) {
    check(nn_fc_skinny((const void*)a, lda, (const void*)w, ldw, (const float*)bias, (float*)out, ldo, M, N, K, (cudaStream_t)stream),
          "fc_skinny");
  });
  m.def("softmax_response",
        [](uintptr_t logits, int rows, int n, int ld, uintptr_t d_stub, uintptr_t direct_out, size_t resp_stride,
           bool write_argmax, uintptr_t counter, uintptr_t flag, uint32_t flag_value, uintptr_t stream, uintptr_t d_push) {
          check(nn_softmax_response((const float*)logits, rows, n, ld, (const void*)d_stub, (void*)direct_out, resp_stride,
                                    write_argmax ? 1 : 0, (uint32_t*)counter, (uint32_t*)flag, flag_value,
                                    (cudaStream_t)stream, (const void*)d_push),
                "softmax_response");
        },
        py::arg("logits"), py::arg("rows"), py::arg("n"), py::arg("ld"), py::arg("d_stub") = 0, py::arg("direct_out") = 0,
        py::arg("resp_stride") = 0, py::arg("write_argmax") = false, py::arg("counter") = 0, py::arg("flag") = 0,
        py::arg("flag_value") = 0, py::arg("stream") = 0, py::arg("d_push") = 0);
  m.def("layernorm",
        [](uintptr_t x, uintptr_t residual, uintptr_t gamma, uintptr_t beta, uintptr_t y, int rows, int hidden, float eps,
           uintptr_t stream) {
          check(nn_layernorm((const void*)x, (const void*)residual, (const float*)gamma, (const float*)beta, (void*)y, rows,
                             hidden, eps, (cudaStream_t)stream),
                "layernorm");
        });
  m.def("bert_embed_ln",
        [](uintptr_t d_stub, uintptr_t direct_ids, size_t req_stride, int batch, int seq, uintptr_t word, uintptr_t pos,
           uintptr_t type, uintptr_t gamma, uintptr_t beta, uintptr_t y, int hidden, int vocab, float eps, uintptr_t stream) {
          check(nn_bert_embed_ln((const void*)d_stub, (const int*)direct_ids, req_stride, batch, seq, (const void*)word,
                                 (const void*)pos, (const void*)type, (const float*)gamma, (const float*)beta, (void*)y,
                                 hidden, vocab, eps, (cudaStream_t)stream),
                "bert_embed_ln");
        });
  m.def("attention_tc",
        [](uintptr_t qk, int ld_qk, uintptr_t vt, int ld_vt, uintptr_t out, int ld_out, uintptr_t v_bias, int batch, int seq,
           int heads, uintptr_t status, uintptr_t stream) {
          check(nn_attention_tc((const void*)qk, ld_qk, (const void*)vt, ld_vt, (void*)out, ld_out, (const float*)v_bias, batch,
                                seq, heads, (uint32_t*)status, (cudaStream_t)stream),
                "attention_tc");
        });
  m.def("attention_d64",
        [](uintptr_t qkv, uintptr_t out, int batch, int seq, int heads, int ld_qkv, int q_off, int k_off, int v_off,
           int ld_out, uintptr_t stream) {
          check(nn_attention_d64((const void*)qkv, (void*)out, batch, seq, heads, ld_qkv, q_off, k_off, v_off, ld_out,
                                 (cudaStream_t)stream),
                "attention_d64");
        });
}

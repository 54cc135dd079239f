// Python bindings of the host core: wire format, pools, transports, server,
// load generator, CPU/GPU apps and the local (no network) benchmark.
#include <pybind11/functional.h>
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "cuda/apps_gpu.h"
#include "host/apps_cpu.h"
#include "host/copy_path_runner.h"
#include "host/dpdk_port.h"
#include "host/loadgen.h"
#include "host/loadgen_compat.h"
#include "host/p2p_rpc_compat.h"
#include "host/splitrpc_server.h"

namespace py = pybind11;

void bind_ops(py::module_& m);  // bindings_ops.cpp

namespace {

py::bytes hdr_bytes(const p2p_rpc_hdr& h) { return py::bytes(reinterpret_cast<const char*>(&h), RPC_HEADER_LEN); }

p2p_rpc_hdr hdr_from(const std::string& b) {
  if (b.size() != RPC_HEADER_LEN) throw std::invalid_argument("header must be 64 bytes");
  p2p_rpc_hdr h;
  std::memcpy(&h, b.data(), RPC_HEADER_LEN);
  return h;
}

py::dict parse_header(const std::string& b) {
  p2p_rpc_hdr h = hdr_from(b);
  py::dict d;
  d["dst_mac"] = mac_to_string(get_eth_header(&h)->dst_mac_);
  d["src_mac"] = mac_to_string(get_eth_header(&h)->src_mac_);
  d["eth_type"] = ntohs(get_eth_header(&h)->eth_type_);
  d["src_ip"] = ipv4_to_string(get_ip_header(&h)->src_ip);
  d["dst_ip"] = ipv4_to_string(get_ip_header(&h)->dst_ip);
  d["ip_tot_len"] = ntohs(get_ip_header(&h)->tot_len);
  d["ip_proto"] = get_ip_header(&h)->protocol;
  d["src_port"] = ntohs(get_udp_header(&h)->src_port);
  d["dst_port"] = ntohs(get_udp_header(&h)->dst_port);
  d["udp_len"] = ntohs(get_udp_header(&h)->len);
  d["udp_check"] = (uint16_t)get_udp_header(&h)->check;
  d["req_token"] = (uint64_t)h.req_token;
  d["sock_perf_header"] = (int64_t)h.sock_perf_header;
  d["seq_num"] = (uint16_t)h.seq_num;
  return d;
}

// A transport port plus whatever owns it.
struct PortHolder {
  Transport* port = nullptr;
  std::shared_ptr<void> owner;
};

struct LoopbackPair {
  std::shared_ptr<LoopbackPort> server, client;
  std::string server_mem;
};

ArenaMem make_arena(const std::string& kind, size_t bytes) {
  if (kind == "malloc") return make_malloc_arena(bytes);
  if (kind == "pinned") {
    const SrpcDeviceOps* ops = srpc_cuda_ops();
    void *h = nullptr, *d = nullptr;
    if (!ops || ops->host_alloc_mapped(bytes, &h, &d) != 0)
      throw std::runtime_error("pinned arena needs a working CUDA device");
    ArenaMem m;
    m.host = (uint8_t*)h;
    m.dev = (uint8_t*)d;
    m.bytes = bytes;
    m.gpu_visible = true;
    m.release = [ops, h] { ops->host_free(h); };
    return m;
  }
  if (kind == "shm" || kind == "shm_pinned") {
    // A memfd mapping that other processes can map too; "shm_pinned" also registers it with CUDA so that GPUs (of
    // every process that registers its own mapping) can read and write it.
    auto* sm = new SrpcSharedMem;
    if (!srpc_shm_create(bytes, kind == "shm_pinned", sm)) {
      delete sm;
      throw std::runtime_error("shared arena: memfd mapping or CUDA registration failed");
    }
    std::memset(sm->host, 0, sm->bytes);
    ArenaMem m;
    m.host = (uint8_t*)sm->host;
    m.dev = (uint8_t*)sm->dev;
    m.bytes = bytes;
    m.fd = sm->fd;
    m.gpu_visible = sm->registered;
    m.release = [sm] {
      srpc_shm_free(sm);
      delete sm;
    };
    return m;
  }
  throw std::invalid_argument("arena kind must be 'malloc', 'pinned', 'shm' or 'shm_pinned'");
}

// ---- apps
struct PyAppState {
  py::function run;
  size_t req_size, resp_size;
};

int py_app_run(AppCtx* c) {
  PyAppState* s = static_cast<PyAppState*>(c->app_ctx_internal);
  py::gil_scoped_acquire gil;
  try {
    s->run((uintptr_t)c->h_stub->req, (uintptr_t)c->h_stub->resp, c->curr_batch_size, (uintptr_t)c->work_stream,
           (uintptr_t)c->d_stub);
  } catch (py::error_already_set& e) {
    srpc_log(SRPC_LOG_ERROR, "python app raised: %s", e.what());
    return 0;
  }
  return 1;
}
int py_app_cleanup(AppCtx* c) {
  PyAppState* s = static_cast<PyAppState*>(c->app_ctx_internal);
  py::gil_scoped_acquire gil;
  delete s;
  c->app_ctx_internal = nullptr;
  return 1;
}
int cpu_app_cleanup(AppCtx* c) {
  delete cpu_state(c);
  c->app_ctx_internal = nullptr;
  return 1;
}

struct AppHolder {
  std::unique_ptr<P2pRpcAppInfo> info;
  std::unique_ptr<P2pRpcSgEngine> engine;
  std::string name;
  void* graph_internal = nullptr;  // state of a graph app (owned by the app's cleanup callback)
};

struct CopyPathHolder {
  std::shared_ptr<AppHolder> app;
  std::unique_ptr<CopyPathBatcher> batcher;
};

std::vector<std::vector<float>> to_weights(const std::vector<py::array_t<float, py::array::c_style | py::array::forcecast>>& ws) {
  std::vector<std::vector<float>> out;
  for (auto& a : ws) out.emplace_back(a.data(), a.data() + a.size());
  return out;
}

std::unique_ptr<P2pRpcSgEngine> make_engine(const std::string& kind, int device, int copy_type) {
  if (kind == "zc") return std::make_unique<P2pRpcSgZcEngine>();
  if (kind == "cpu") return std::make_unique<P2pRpcSgCpuEngine>();
  if (kind == "gpu") {
    P2pRpcSgEngine* e = srpc_make_gpu_sg_engine(device, copy_type);
    if (!e) throw std::runtime_error("GPU scatter-gather engine needs a CUDA device");
    return std::unique_ptr<P2pRpcSgEngine>(e);
  }
  throw std::invalid_argument("engine must be 'zc', 'cpu' or 'gpu'");
}

std::shared_ptr<AppHolder> make_app(const std::string& name, int device, size_t req_size, size_t resp_size,
                                    const std::vector<py::array_t<float, py::array::c_style | py::array::forcecast>>& weights,
                                    int pool_size, int launch_type, int batch, const std::string& engine, int copy_type) {
  auto h = std::make_shared<AppHolder>();
  h->name = name;
  auto w = to_weights(weights);
  if (device < 0) {
    auto* s = new CpuAppState;
    s->req_size = req_size;
    s->resp_size = resp_size;
    s->weights = std::move(w);
    AppRunCB run = nullptr;
    if (name == "echo") run = cpu_echo_run;
    else if (name == "vec_add") run = cpu_vec_add_run;
    else if (name == "matmul") run = cpu_mm_run;
    else if (name == "lenet5") run = cpu_lenet5_run;
    else if (name == "lenet_ref") run = cpu_lenet_ref_run;
    else if (name == "lstm") run = cpu_lstm_run;
    if (!run) {
      delete s;
      throw std::invalid_argument("unknown CPU app '" + name + "'");
    }
    h->info.reset(new P2pRpcAppInfo(cpu_app_noop, run, cpu_app_cleanup, cpu_app_noop, -1, req_size, resp_size, pool_size,
                                    s, launch_type, batch));
  } else {
    GpuAppHandle g = srpc_make_gpu_app(name.c_str(), device, req_size, resp_size, w);
    if (!g.run) throw std::runtime_error("GPU app '" + name + "' unavailable (unknown name or no CUDA device)");
    h->info.reset(new P2pRpcAppInfo(g.init, g.run, g.cleanup, g.complete, device, req_size, resp_size, pool_size,
                                    g.internal, launch_type, batch));
  }
  h->engine = make_engine(engine.empty() ? (device < 0 ? "cpu" : "gpu") : engine, device, copy_type);
  return h;
}

std::shared_ptr<AppHolder> make_python_app(py::function run, int device, size_t req_size, size_t resp_size, int pool_size,
                                           int launch_type, int batch, const std::string& engine, int copy_type) {
  auto h = std::make_shared<AppHolder>();
  h->name = "python";
  auto* s = new PyAppState{std::move(run), req_size, resp_size};
  h->info.reset(new P2pRpcAppInfo(cpu_app_noop, py_app_run, py_app_cleanup, cpu_app_noop, device, req_size, resp_size,
                                  pool_size, s, launch_type, batch));
  h->engine = make_engine(engine.empty() ? (device < 0 ? "cpu" : "gpu") : engine, device, copy_type);
  return h;
}

std::shared_ptr<AppHolder> make_graph_app(int device, size_t req_size, size_t resp_size, int pool_size, int batch,
                                          const std::string& engine, int copy_type) {
  auto h = std::make_shared<AppHolder>();
  h->name = "graph";
  GpuAppHandle g = srpc_make_graph_app();
  h->graph_internal = g.internal;
  h->info.reset(new P2pRpcAppInfo(g.init, g.run, g.cleanup, g.complete, device, req_size, resp_size, pool_size, g.internal,
                                  4, batch));
  h->engine = make_engine(engine.empty() ? "gpu" : engine, device, copy_type);
  return h;
}

// Members are destroyed in reverse order: the server (and its threads) goes
// first, then the apps it was running, then the port.
struct ServerHolder {
  PortHolder port;
  std::vector<std::shared_ptr<AppHolder>> apps;
  std::vector<std::unique_ptr<NvlRemoteReplica>> remotes;  // outlive the server's threads (declared before `server`)
  std::unique_ptr<SplitRpcServer> server;
};

// A batched server and the app it serves.
struct BatchedServerHolder {
  std::shared_ptr<AppHolder> app;
  std::unique_ptr<NvlBatchedServer> server;
};

struct ClientHolder {
  PortHolder port;
  std::unique_ptr<P2pRpcAppClient> client;
};

app_req_cb req_cb_by_name(const std::string& k) {
  if (k == "echo") return echo_fill;
  if (k == "vec_add") return vec_add_fill;
  if (k == "const5") return const_float_fill;
  if (k == "uniform") return uniform_float_fill;
  if (k == "normal") return normal_float_fill;
  if (k == "ids") return token_ids_fill;
  throw std::invalid_argument("payload kind must be echo, vec_add, const5, uniform, normal or ids");
}
app_resp_cb resp_cb_by_name(const std::string& k) {
  if (k == "echo") return echo_check;
  if (k == "vec_add") return vec_add_check;
  return nullptr;
}

}  // namespace

PYBIND11_MODULE(_C, m) {
  m.doc() = "splitrpc_b200 native core";
  m.attr("RPC_HEADER_LEN") = (int)RPC_HEADER_LEN;
  m.attr("UDP_HEADER_LEN") = (int)UDP_HEADER_LEN;
  m.attr("RPC_HEADER_TAIL_LEN") = (int)RPC_HEADER_TAIL_LEN;
  m.attr("MAX_BI_SIZE") = (int)MAX_BI_SIZE;
  m.def("rpc_mtu", [] { return rpc_mtu(); });
  m.def("set_rpc_mtu", [](size_t v) { set_rpc_mtu(v); });
  m.def("set_log_level", [](int l) { srpc_set_log_level(l); });
  m.def("read_env_int", [](const std::string& n, long d) { return readEnvInfo<long>(n.c_str(), d); });
  m.def("cuda_available", [] {
    const SrpcDeviceOps* o = srpc_cuda_ops();
    return o && o->device_count() > 0;
  });

  // ---- wire
  m.def("client_conn_template", [](const std::string& uri) {
    p2p_rpc_conn_info* c = initialize_client_conn_info(uri);
    if (!c) throw std::invalid_argument("bad client URI");
    py::bytes b = hdr_bytes(c->hdr_template);
    release_conn_info(c);
    return b;
  });
  m.def("server_conn_template", [](const std::string& uri) {
    p2p_rpc_conn_info* c = initialize_src_conn_info(uri);
    if (!c) throw std::invalid_argument("bad server URI");
    py::bytes b = hdr_bytes(c->hdr_template);
    release_conn_info(c);
    return b;
  });
  m.def("reply_template", [](const std::string& server_tmpl, const std::string& recv_hdr) {
    p2p_rpc_conn_info c;
    c.hdr_template = hdr_from(server_tmpl);
    p2p_rpc_hdr r = hdr_from(recv_hdr);
    set_conn_info(&c, &r);
    return hdr_bytes(c.hdr_template);
  });
  m.def("parse_header", &parse_header);
  m.def("build_fragments",
        [](const std::string& tmpl, uint64_t token, const std::string& payload, size_t mtu, bool is_reply) {
          p2p_rpc_conn_info c;
          c.hdr_template = hdr_from(tmpl);
          py::list out;
          size_t n = num_fragments(payload.size(), mtu), left = payload.size();
          for (size_t i = 0; i < n; i++) {
            size_t len = left < mtu ? left : mtu;
            p2p_rpc_hdr h;
            fill_frag_hdr(&h, &c, token, (uint16_t)i, (uint16_t)len, is_reply);
            out.append(py::make_tuple(hdr_bytes(h), py::bytes(payload.data() + i * mtu, len)));
            left -= len;
          }
          return out;
        },
        py::arg("conn_template"), py::arg("token"), py::arg("payload"), py::arg("mtu"), py::arg("is_reply") = false);
  m.def("swap_header", [](const std::string& b) {
    p2p_rpc_hdr h = hdr_from(b);
    swap_eth_hdr(&h);
    add_udp_cksum(&h);
    return hdr_bytes(h);
  });
  m.def("ipv4_pseudo_csum", [](const std::string& b) {
    p2p_rpc_hdr h = hdr_from(b);
    return ipv4_pseudo_csum(get_ip_header(&h));
  });
  m.def("ipv4_header_csum", [](const std::string& b) {
    p2p_rpc_hdr h = hdr_from(b);
    return ipv4_header_csum(get_ip_header(&h));
  });
  m.def("num_fragments", &num_fragments);

  // ---- stats
  m.def("percentile", [](std::vector<uint64_t> v, double p) { return getPercentile(v, p); });
  m.def("mean", [](const std::vector<uint64_t>& v) { return getMean(v); });
  m.def("format_stat", [](const std::string& k, const std::vector<uint64_t>& v) { return format_stat(k, v); });

  // ---- tring
  py::class_<P2pRpcTring>(m, "P2pRpcTring")
      .def(py::init([](uintptr_t base, size_t cap) { return new P2pRpcTring((void*)base, cap); }))
      .def("get_next", [](P2pRpcTring& t, size_t n) { return (uintptr_t)t.get_next(n); })
      .def_property_readonly("offset", &P2pRpcTring::offset);

  // ---- copy-list builders (addresses are plain integers)
  m.def("gather_list", [](const std::vector<std::pair<uintptr_t, size_t>>& frags, uintptr_t dst) {
    auto bufs = std::make_unique<p2p_bufs>();
    auto skb = std::make_unique<p2p_sk_buf>();
    bufs->num_items = (uint16_t)frags.size();
    for (size_t i = 0; i < frags.size(); i++) {
      bufs->burst_items[i] = frags[i].first;
      bufs->item_size[i] = frags[i].second;
    }
    gather_skbs(skb.get(), bufs.get(), (uint8_t*)dst);
    std::vector<std::tuple<uintptr_t, uintptr_t, size_t>> out;
    for (size_t i = 0; i < skb->num_items; i++) out.emplace_back(skb->i_buf[i], skb->o_buf[i], skb->len[i]);
    return out;
  });
  m.def("scatter_list", [](const std::vector<std::pair<uintptr_t, size_t>>& frags, uintptr_t src) {
    auto bufs = std::make_unique<p2p_bufs>();
    auto skb = std::make_unique<p2p_sk_buf>();
    bufs->num_items = (uint16_t)frags.size();
    for (size_t i = 0; i < frags.size(); i++) {
      bufs->burst_items[i] = frags[i].first;
      bufs->item_size[i] = frags[i].second;
    }
    scatter_skbs(skb.get(), bufs.get(), (uint8_t*)src);
    std::vector<std::tuple<uintptr_t, uintptr_t, size_t>> out;
    for (size_t i = 0; i < skb->num_items; i++) out.emplace_back(skb->i_buf[i], skb->o_buf[i], skb->len[i]);
    return out;
  });

  // Multi-tensor pack list of one request: frags = [(addr, len)], tensors = [(batch_base_addr, tensor_bytes)].
  m.def("pack_list", [](const std::vector<std::pair<uintptr_t, size_t>>& frags,
                        const std::vector<std::pair<uintptr_t, size_t>>& tensors, int batch_index) {
    auto bufs = std::make_unique<p2p_bufs>();
    auto skb = std::make_unique<p2p_sk_buf>();
    bufs->num_items = (uint16_t)frags.size();
    for (size_t i = 0; i < frags.size(); i++) {
      bufs->burst_items[i] = frags[i].first;
      bufs->item_size[i] = frags[i].second;
    }
    g_params_v2 stub{};
    if (tensors.size() > MAX_NUM_TENSORS) throw std::invalid_argument("at most 4 tensors per request");
    for (size_t k = 0; k < tensors.size(); k++) {
      stub.inputs[k] = tensors[k].first;
      stub.input_tensor_size[k] = tensors[k].second;
    }
    gather_skbs_v2(skb.get(), bufs.get(), &stub, (int)tensors.size(), batch_index);
    std::vector<std::tuple<uintptr_t, uintptr_t, size_t>> out;
    for (size_t i = 0; i < skb->num_items; i++) out.emplace_back(skb->i_buf[i], skb->o_buf[i], skb->len[i]);
    return out;
  });

  // ---- reassembly harness: feeds (header, payload) pairs through the pool and the CPU engine
  struct Reassembler {
    P2pRpcRRPool pool;
    P2pRpcSgCpuEngine eng;
    std::vector<std::unique_ptr<std::string>> keep;
    size_t req_size;
    Reassembler(size_t req, int pool_size) : pool(pool_size), req_size(req) {
      p2p_rpc_conn_info* c = initialize_src_conn_info("b8:ce:f6:cc:6a:52,192.168.25.1,50051");
      pool.setup_and_init_rr_pool(c, req);
      release_conn_info(c);
    }
  };
  py::class_<Reassembler>(m, "Reassembler")
      .def(py::init<size_t, int>(), py::arg("req_size"), py::arg("pool_size") = 64)
      .def("feed",
           [](Reassembler& r, const std::string& hdr, const std::string& payload) -> py::object {
             p2p_rpc_hdr h = hdr_from(hdr);
             r.keep.emplace_back(new std::string(payload));
             const std::string& kept = *r.keep.back();
             P2pRpcRr* rr = r.pool.append_to_rr(&h, 1, (uintptr_t)kept.data(), kept.size());
             if (!rr) return py::none();
             if (!rr->is_rr_ready()) return py::none();
             r.pool.mark_rx_ready_rr(rr);
             P2pRpcRr* ready = r.pool.get_next_rx_ready_rr();
             std::string out(r.req_size, '\0');
             g_params p{(uint8_t*)out.data(), nullptr};
             r.eng.gather(ready, &p);
             uint64_t tok = ready->req_token;
             size_t runs = ready->payload_sk_bufs->num_items;
             r.pool.reap_rr(ready);
             return py::make_tuple(tok, py::bytes(out), runs);
           })
      .def("expire", [](Reassembler& r, uint64_t timeout_ns) { return r.pool.expire_stale(getCurNs(), timeout_ns, nullptr); })
      .def_property_readonly("partial", [](Reassembler& r) { return r.pool.num_partial(); })
      .def_property_readonly("counters", [](Reassembler& r) {
        const RrPoolCounters& c = r.pool.counters();
        py::dict d;
        d["allocated"] = c.allocated;
        d["grown"] = c.grown;
        d["dropped_zero_token"] = c.dropped_zero_token;
        d["dropped_bad_seq"] = c.dropped_bad_seq;
        d["dropped_dup"] = c.dropped_dup;
        d["expired"] = c.expired;
        d["rx_ready"] = c.rx_ready;
        d["reaped"] = c.reaped;
        return d;
      });

  // ---- transports
  py::class_<PortHolder>(m, "Port")
      .def_property_readonly("name", [](PortHolder& p) { return std::string(p.port->name()); })
      .def_property_readonly("counters", [](PortHolder& p) {
        py::dict d;
        TransportCounters& c = p.port->counters;
        d["rx_pkts"] = c.rx_pkts.load();
        d["tx_pkts"] = c.tx_pkts.load();
        d["rx_bytes"] = c.rx_bytes.load();
        d["tx_bytes"] = c.tx_bytes.load();
        d["tx_dropped"] = c.tx_dropped.load();
        d["arena_full"] = c.arena_full.load();
        d["injected_faults"] = c.injected_faults.load();
        return d;
      });

  m.def("make_loopback_pair",
        [](size_t slot_bytes, size_t n_slots, const std::string& server_mem) {
          // the receive rings hold every packet that can be in flight (the caller sizes n_slots for that)
          const size_t depth = std::max<size_t>(65536, n_slots);
          auto srv = std::make_shared<LoopbackPort>(make_arena(server_mem, slot_bytes * n_slots),
                                                    make_arena(server_mem, slot_bytes * n_slots), slot_bytes, depth);
          auto cli = std::make_shared<LoopbackPort>(make_malloc_arena(slot_bytes * n_slots),
                                                    make_malloc_arena(slot_bytes * n_slots), slot_bytes, depth);
          LoopbackPort::connect(srv.get(), cli.get());
          // Buffers that the client fills and hands over by reference are made of the same kind of memory as the
          // server's receive arena (so a shared arena comes with shared by-reference buffers).
          if (server_mem != "malloc") srv->set_region_factory([server_mem](size_t bytes) { return make_arena(server_mem, bytes); });
          // Each port keeps the other alive, since it delivers into its arenas.
          auto both = std::make_shared<std::pair<std::shared_ptr<LoopbackPort>, std::shared_ptr<LoopbackPort>>>(srv, cli);
          PortHolder s{srv.get(), both}, c{cli.get(), both};
          return py::make_tuple(s, c);
        },
        py::arg("slot_bytes"), py::arg("n_slots") = 4096, py::arg("server_mem") = "malloc");
  // A buffer of the receiving port's kind of memory that the sender fills and hands over by reference: returns
  // (host address, device address, bytes, index among the receiving port's payload regions).
  m.def("alloc_dma_region", [](PortHolder& sender, size_t bytes) {
    DmaRegion r;
    if (!sender.port->alloc_dma_region(bytes, &r)) throw std::runtime_error("this port has no shareable by-reference memory");
    auto* lp = dynamic_cast<LoopbackPort*>(sender.port);
    DmaRegion all[NVL_MAX_REGIONS];
    int n = lp && lp->peer() ? lp->peer()->dma_regions(all, NVL_MAX_REGIONS) : 0;
    return py::make_tuple((uintptr_t)r.host_base, (uintptr_t)r.dev_base, (size_t)r.bytes, n - 1);
  });
  // Copy lanes of the emulated NIC DMA of a loopback port (threads that write the fragments of a burst into the peer's
  // receive arena; 1 = the sending thread alone).
  m.def("set_loopback_dma_lanes", [](PortHolder& p, int lanes) {
    auto* lp = dynamic_cast<LoopbackPort*>(p.port);
    if (!lp) throw std::invalid_argument("not a loopback port");
    lp->set_dma_lanes(lanes);
  }, py::arg("port"), py::arg("lanes"));
  m.def("set_loopback_faults",
        [](PortHolder& p, double drop, double dup, double reorder, double truncate, bool zero_token, int force_seq,
           uint64_t seed) {
          auto* lp = dynamic_cast<LoopbackPort*>(p.port);
          if (!lp) throw std::invalid_argument("not a loopback port");
          LoopbackFaults f;
          f.drop = drop;
          f.duplicate = dup;
          f.reorder = reorder;
          f.truncate = truncate;
          f.zero_token = zero_token;
          f.force_seq = force_seq;
          f.seed = seed;
          lp->set_faults(f);
        },
        py::arg("port"), py::arg("drop") = 0.0, py::arg("duplicate") = 0.0, py::arg("reorder") = 0.0,
        py::arg("truncate") = 0.0, py::arg("zero_token") = false, py::arg("force_seq") = -1, py::arg("seed") = 99);
  m.def("make_udp_port",
        [](const std::string& ip, int port, size_t slot_bytes, size_t n_slots, const std::string& dst_ip, int dst_port,
           const std::string& mem) {
          auto u = std::make_shared<UdpPort>(ip.c_str(), port, slot_bytes, make_arena(mem, slot_bytes * n_slots),
                                             make_arena(mem, slot_bytes * n_slots));
          if (!u->ok()) throw std::runtime_error("UDP bind failed");
          if (!dst_ip.empty()) u->set_destination(dst_ip.c_str(), dst_port);
          return py::make_tuple(PortHolder{u.get(), u}, u->bound_port());
        },
        py::arg("ip"), py::arg("port"), py::arg("slot_bytes"), py::arg("n_slots") = 4096, py::arg("dst_ip") = "",
        py::arg("dst_port") = 0, py::arg("mem") = "malloc");
#ifdef SPLITRPC_HAVE_DPDK
  m.def("dpdk_available", [] { return true; });
  // A port of NIC `nic_port` with header/data split into arenas of kind `mem` (see make_loopback_pair).
  m.def("make_dpdk_port",
        [](int nic_port, int queue_id, size_t slot_bytes, size_t n_slots, const std::string& mem) {
          Transport* t = srpc_open_dpdk_port(nic_port, queue_id, slot_bytes, n_slots, [mem](size_t b) { return make_arena(mem, b); });
          if (!t) throw std::runtime_error("DPDK port could not be opened");
          std::shared_ptr<Transport> owner(t);
          return PortHolder{t, owner};
        },
        py::arg("nic_port") = 0, py::arg("queue_id") = 0, py::arg("slot_bytes") = 8192, py::arg("n_slots") = 4096,
        py::arg("mem") = "shm_pinned");
#else
  m.def("dpdk_available", [] { return false; });
  m.def("make_dpdk_port", [](py::args, py::kwargs) -> PortHolder {
    throw std::runtime_error("this build has no DPDK (build with SPLITRPC_WITH_DPDK=1 on a machine with libdpdk and a NIC)");
  });
#endif

  // ---- apps
  py::class_<AppHolder, std::shared_ptr<AppHolder>>(m, "App")
      .def_property_readonly("name", [](AppHolder& a) { return a.name; })
      .def_property_readonly("init_ok", [](AppHolder& a) { return a.info->init_ok; })
      .def_property_readonly("work_stream", [](AppHolder& a) { return (uintptr_t)a.info->app_ctx->work_stream; })
      .def_property_readonly("d_stub", [](AppHolder& a) { return (uintptr_t)a.info->app_ctx->d_stub; })
      .def_property_readonly("req_ring", [](AppHolder& a) {
        auto* mp = a.info->app_rr_pool->rr_mem_pool;
        return py::make_tuple((uintptr_t)mp->get_req_addr_range(), mp->get_req_addr_pool_size(), mp->is_double_mapped());
      })
      // Gathers into this app's request ring deserialise ResNet images on the way (fp32 CHW -> normalised bf16
      // space-to-depth, see sg_kernels.cuh); an empty mean list switches back to plain copies.  The caller zeroes the
      // ring once before the first request.
      .def("set_ingress_stem_s2d",
           [](AppHolder& a, std::vector<float> mean, std::vector<float> inv_std) {
             auto* mp = a.info->app_rr_pool->rr_mem_pool;
             if (mean.empty()) return a.engine->set_gather_transform(SG_TRANSFORM_NONE, 0, 0, nullptr) == 0;
             if (mean.size() != 3 || inv_std.size() != 3) throw std::invalid_argument("mean / inv_std need 3 values");
             float params[6] = {mean[0], mean[1], mean[2], inv_std[0], inv_std[1], inv_std[2]};
             return a.engine->set_gather_transform(SG_TRANSFORM_STEM_S2D, (uint64_t)(uintptr_t)mp->get_req_addr_range(),
                                                   (uint32_t)a.info->app_rr_pool->req_size, params) == 0;
           })
      .def_property_readonly("resp_ring", [](AppHolder& a) {
        auto* mp = a.info->app_rr_pool->rr_mem_pool;
        return py::make_tuple((uintptr_t)mp->get_resp_addr_range(), mp->get_resp_addr_pool_size(), mp->is_double_mapped());
      })
      .def("capture_begin",
           [](AppHolder& a) {
             if (int e = srpc_capture_begin(a.info->app_ctx->work_stream)) throw std::runtime_error("capture_begin: CUDA error " + std::to_string(e));
           })
      .def("capture_end",
           [](AppHolder& a, int batch) {
             if (!a.graph_internal) throw std::runtime_error("capture_end: not a graph app");
             cudaGraphExec_t exec = nullptr;
             if (int e = srpc_capture_end(a.info->app_ctx->work_stream, &exec)) throw std::runtime_error("capture_end: CUDA error " + std::to_string(e));
             srpc_graph_app_set(a.graph_internal, batch, exec);
           })
      .def("sync", [](AppHolder& a) { return a.info->app_ctx->WaitForAppRunComplete(); })
      // Device address of the app's response-push block: kernels given it store responses where the ingress asked
      // for them and complete the slots themselves once the server has enabled that (see RespPushCtx).
      .def_property_readonly("d_push", [](AppHolder& a) { return (uintptr_t)a.info->app_ctx->d_push; })
      // Tells the worker that the app's own kernels take d_push (no separate push kernel is queued behind them).
      .def("set_self_push", [](AppHolder& a, bool on) { a.info->app_ctx->self_push = on; })
      .def_property_readonly("completion_by_device", [](AppHolder& a) { return a.info->completion_by_device; })
      // Writes the slot index of the batch's first request into the push block (stand-alone timing loops; the server's
      // workers do this themselves).
      .def("set_first_slot", [](AppHolder& a, uint32_t slot) {
        a.info->app_ctx->h_push->first_slot = slot;
        std::atomic_thread_fence(std::memory_order_seq_cst);
        a.info->stage_window((int)slot, 0, false);
      })
      // Stream-ordered update of what the next batch's kernels read (stand-alone timing loops; the server's workers do
      // this themselves): the stub points at req / resp, the batch of `batch` requests starts at `first_slot`.  With
      // `armed` the transmit offsets are read from the slot table when the update runs (queue it behind the doorbell
      // wait), otherwise they are taken from the table now.
      .def("stage_window",
           [](AppHolder& a, uintptr_t req, uintptr_t resp, int first_slot, int batch, bool armed) {
             a.info->app_ctx->h_stub->req = (uint8_t*)req;
             a.info->app_ctx->h_stub->resp = (uint8_t*)resp;
             a.info->app_ctx->h_push->first_slot = (uint32_t)first_slot;
             std::atomic_thread_fence(std::memory_order_seq_cst);
             a.info->stage_window(first_slot, batch, armed);
           },
           py::arg("req"), py::arg("resp"), py::arg("first_slot"), py::arg("batch"), py::arg("armed") = false)
      // Queues `n` runs of the app on the window of `batch` requests that starts at slot 0, back to back on the work
      // stream, and returns without waiting: for device-side timing with events recorded on `work_stream` around it.
      .def("queue_runs",
           [](AppHolder& a, int batch, int n) {
             AppCtx* c = a.info->app_ctx;
             c->curr_batch_size = batch;
             *c->h_stub = *a.info->app_rr_pool->get_app_rr(0)->h_stub;
             c->h_push->first_slot = 0;
             std::atomic_thread_fence(std::memory_order_seq_cst);
             for (int i = 0; i < n; i++) {
               a.info->stage_window(0, batch, false);
               a.info->app_run(c);
             }
           },
           py::arg("batch"), py::arg("n"))
      .def_property_readonly("pool_size", [](AppHolder& a) { return a.info->app_rr_pool->get_pool_size(); })
      // Slot-level access for stand-alone timing loops and tests (the server's threads do all of this themselves):
      // device-side address of the slot state words, state and response destination of one slot, and a reset of the
      // whole ring (every slot FREE, no destinations, ring addresses from the start).
      .def_property_readonly("states_dev", [](AppHolder& a) { return (uintptr_t)a.info->app_rr_pool->rr_mem_pool->get_doorbells_device(); })
      .def_property_readonly("d_first_slot", [](AppHolder& a) { return (uintptr_t)&a.info->app_ctx->d_push->first_slot; })
      .def("slot_state", [](AppHolder& a, int i) { return (uint32_t)__atomic_load_n(a.info->app_rr_pool->get_app_rr(i)->h_state, __ATOMIC_ACQUIRE); })
      .def("set_slot_state", [](AppHolder& a, int i, uint32_t v) { __atomic_store_n(a.info->app_rr_pool->get_app_rr(i)->h_state, v, __ATOMIC_RELEASE); })
      .def("set_tx_off", [](AppHolder& a, int i, uint64_t off) { __atomic_store_n(a.info->app_rr_pool->get_app_rr(i)->h_tx_off, off, __ATOMIC_RELEASE); })
      .def("reset_slots", [](AppHolder& a) {
        P2pRpcAppRrPool* pool = a.info->app_rr_pool;
        pool->init_pool();
        a.info->consumer_seq = 0;
        for (int i = 0; i < pool->get_pool_size(); i++) {
          __atomic_store_n(pool->get_app_rr(i)->h_tx_off, P2pRpcAppRrMemPool::kNoTxOffset, __ATOMIC_RELAXED);
          __atomic_store_n(pool->get_app_rr(i)->h_state, (uint32_t)APP_RR_STATUS::FREE, __ATOMIC_RELEASE);
        }
      })
      // Completion by the serving side, set up by hand (the server does this in add_replica): responses go to
      // tx_base + the slot's offset, tx_base being this process's device-side address of the transmit arena.
      .def("enable_device_completion", [](AppHolder& a, uintptr_t tx_base, uint64_t tx_bytes) { a.info->enable_device_completion(tx_base, tx_bytes); })
      .def("disable_device_completion", [](AppHolder& a) { a.info->disable_device_completion(); })
      .def_property_readonly("exportable", [](AppHolder& a) { return a.info->app_rr_pool->rr_mem_pool->exportable(); })
      // Points the app's stub at explicit addresses (default: the start of both rings),
      // e.g. before a warm-up run or a stand-alone timing loop.
      .def("set_stub",
           [](AppHolder& a, uintptr_t req, uintptr_t resp) {
             auto* mp = a.info->app_rr_pool->rr_mem_pool;
             a.info->app_ctx->h_stub->req = req ? (uint8_t*)req : (uint8_t*)mp->get_req_addr_range();
             a.info->app_ctx->h_stub->resp = resp ? (uint8_t*)resp : (uint8_t*)mp->get_resp_addr_range();
             std::atomic_thread_fence(std::memory_order_seq_cst);
             a.info->stage_window((int)a.info->app_ctx->h_push->first_slot, 0, false);
           },
           py::arg("req") = 0, py::arg("resp") = 0)
      // Runs the app once for `batch` requests at the current stub without waiting.
      .def("launch",
           [](AppHolder& a, int batch) {
             a.info->app_ctx->curr_batch_size = batch;
             if (!a.info->app_run(a.info->app_ctx)) throw std::runtime_error("app run failed");
           })
      .def_property_readonly("sg_counters", [](AppHolder& a) {
        py::dict d;
        d["gathers"] = a.engine->counters.gathers;
        d["scatters"] = a.engine->counters.scatters;
        d["items"] = a.engine->counters.items;
        d["bytes"] = a.engine->counters.bytes;
        d["timeouts"] = a.engine->counters.timeouts;
        d["engine"] = std::string(a.engine->name());
        return d;
      });
  m.def("make_app", &make_app, py::arg("name"), py::arg("device") = -1, py::arg("req_size") = 1024,
        py::arg("resp_size") = 1024, py::arg("weights") = std::vector<py::array_t<float>>{}, py::arg("pool_size") = 256,
        py::arg("launch_type") = 1, py::arg("batch") = 1, py::arg("engine") = "", py::arg("copy_type") = 2);
  m.def("make_graph_app", &make_graph_app, py::arg("device") = 0, py::arg("req_size") = 1024, py::arg("resp_size") = 1024,
        py::arg("pool_size") = 256, py::arg("batch") = 1, py::arg("engine") = "", py::arg("copy_type") = 2);
  m.def("make_python_app", &make_python_app, py::arg("run"), py::arg("device") = -1, py::arg("req_size") = 1024,
        py::arg("resp_size") = 1024, py::arg("pool_size") = 256, py::arg("launch_type") = 1, py::arg("batch") = 1,
        py::arg("engine") = "", py::arg("copy_type") = 2);

  // Local benchmark without a network: fill slot windows, run do_batch_work_sync
  // `iters` times, return the per-iteration host times in ns (reference
  // src/local_bench/p2p_rpc_local_bench.cc:40-115).
  m.def("local_bench",
        [](std::shared_ptr<AppHolder> app, int iters, int batch, py::object fill) {
          P2pRpcAsyncAppServer srv;
          int idx = srv.register_app(app->info.get());
          P2pRpcAppRrPool* pool = app->info->app_rr_pool;
          pool->init_pool();
          std::vector<uint64_t> ns;
          py::list outs;
          for (int it = 0; it < iters; it++) {
            int first = -1;
            for (int b = 0; b < batch; b++) {
              P2pRpcAppRr* r = pool->get_next();
              if (b == 0) first = r->rr_idx;
              if (!fill.is_none()) fill((uintptr_t)r->h_stub->req, r->req_size, it * batch + b);
            }
            uint64_t t0;
            bool ok;
            {
              py::gil_scoped_release rel;
              t0 = getCurNs();
              ok = srv.do_batch_work_sync(idx, first, batch);
              ns.push_back(getCurNs() - t0);
            }
            if (!ok) throw std::runtime_error("local_bench: bounded wait ran out");
            if (it == iters - 1) outs.append((uintptr_t)pool->get_app_rr(first)->h_stub->resp);
          }
          return py::make_tuple(ns, outs);
        },
        py::arg("app"), py::arg("iters"), py::arg("batch") = 1, py::arg("fill") = py::none());

  // ---- the comparison system's copy path (requests from ordinary host memory, one copy in and out per request)
  py::class_<CopyPathHolder, std::shared_ptr<CopyPathHolder>>(m, "CopyPathBatcher")
      .def(py::init([](std::shared_ptr<AppHolder> app, int max_batch) {
             auto h = std::make_shared<CopyPathHolder>();
             h->app = app;
             h->batcher.reset(new CopyPathBatcher(app->info.get(), max_batch));
             return h;
           }),
           py::arg("app"), py::arg("max_batch") = 1)
      // Blocks (without the interpreter lock) until the request has been through a batch; returns the response.
      .def("submit",
           [](CopyPathHolder& h, py::bytes req) {
             char* data = nullptr;
             Py_ssize_t len = 0;
             if (PyBytes_AsStringAndSize(req.ptr(), &data, &len) != 0) throw py::error_already_set();
             std::string resp(h.batcher->resp_size(), '\0');
             bool ok;
             {
               py::gil_scoped_release rel;
               ok = h.batcher->submit(data, (size_t)len, resp.data());
             }
             if (!ok) throw std::runtime_error("copy path: the batch failed or the worker has stopped");
             return py::bytes(resp);
           })
      .def("times",
           [](CopyPathHolder& h) {
             CopyPathTimes t = h.batcher->times();
             py::dict d;
             d["h2d_ns"] = t.h2d_ns;
             d["run_ns"] = t.run_ns;
             d["d2h_ns"] = t.d2h_ns;
             d["batches"] = t.batches;
             d["requests"] = t.requests;
             return d;
           })
      .def_property_readonly("max_batch", [](CopyPathHolder& h) { return h.batcher->max_batch(); })
      .def("stop", [](CopyPathHolder& h) {
        py::gil_scoped_release rel;
        h.batcher->stop();
      });

  // ---- server
  py::class_<ServerHolder, std::shared_ptr<ServerHolder>>(m, "Server")
      .def(py::init([](PortHolder port, const std::string& uri, size_t req_size, size_t resp_size, int server_mode,
                       int max_batch, int zerocopy, int rr_pool_size, uint64_t reassembly_timeout_ns, int steer_policy,
                       int gather_burst, int device_completion) {
             auto h = std::make_shared<ServerHolder>();
             ServerConfig c;
             if (!uri.empty()) c.server_uri = uri;
             c.req_size = req_size;
             c.resp_size = resp_size;
             c.server_mode = server_mode;
             c.max_batch = max_batch;
             c.zerocopy = zerocopy;
             c.rr_pool_size = rr_pool_size;
             c.reassembly_timeout_ns = reassembly_timeout_ns;
             c.steer_policy = steer_policy;
             c.gather_burst = gather_burst;
             c.device_completion = device_completion;
             h->port = port;
             h->server.reset(new SplitRpcServer(port.port, c));
             return h;
           }),
           py::arg("port"), py::arg("uri") = "", py::arg("req_size") = 1024, py::arg("resp_size") = 1024,
           py::arg("server_mode") = 2, py::arg("max_batch") = 1, py::arg("zerocopy") = 0, py::arg("rr_pool_size") = 1023,
           py::arg("reassembly_timeout_ns") = 200000000ull, py::arg("steer_policy") = 0, py::arg("gather_burst") = 64,
           py::arg("device_completion") = 1)
      .def("add_replica",
           [](ServerHolder& s, std::shared_ptr<AppHolder> app) {
             s.apps.push_back(app);
             return s.server->add_replica(app->info.get(), app->engine.get());
           })
      // Adds a replica served by a BatchedServer in another process (usually another GPU): connects to its control
      // socket, performs the ALLOC handshake (this server's transmit arena travels with it when it is a shared
      // mapping), maps the replica's rings and doorbells, and creates the engine that fills them from
      // `ingress_device` (-1: CPU engine, rings in host memory only).
      .def("add_remote_replica",
           [](ServerHolder& s, const std::string& path, uint32_t func_id, int ingress_device, int copy_type, int timeout_ms, bool pull) {
             std::string err;
             std::unique_ptr<NvlRemoteReplica> r;
             {
               py::gil_scoped_release rel;
               r = NvlRemoteReplica::connect(path, func_id, ingress_device, copy_type, s.server->tx_arena(), timeout_ms, &err,
                                             pull ? s.server->port() : nullptr);
             }
             if (!r) throw std::runtime_error("add_remote_replica: " + err);
             int idx = s.server->add_remote_replica(r.get());
             s.remotes.push_back(std::move(r));
             return idx;
           },
           py::arg("path"), py::arg("func_id") = 1234, py::arg("ingress_device") = -1, py::arg("copy_type") = 2,
           py::arg("timeout_ms") = 10000, py::arg("pull") = false)
      // Transmit arena of the server's port: (host base, device base, bytes, slot bytes).
      .def_property_readonly("tx_arena", [](ServerHolder& s) -> py::tuple {
        const TxArenaInfo* t = s.server->tx_arena();
        if (!t) return py::make_tuple((uintptr_t)0, (uintptr_t)0, (size_t)0, (size_t)0);
        return py::make_tuple((uintptr_t)t->host_base, (uintptr_t)t->dev_base, (size_t)t->bytes, (size_t)t->slot_bytes);
      })
      // This process's mapping of a remote replica's rings and slot words (addresses are valid on the ingress GPU).
      .def("remote_rings",
           [](ServerHolder& s, int remote_idx) {
             P2pRpcAppRrPool* pool = s.remotes.at((size_t)remote_idx)->pool();
             P2pRpcAppRrMemPool* mp = pool->rr_mem_pool;
             py::dict d;
             d["req_base"] = (uintptr_t)mp->get_req_addr_range();
             d["req_capacity"] = mp->get_req_addr_pool_size();
             d["resp_base"] = (uintptr_t)mp->get_resp_addr_range();
             d["resp_capacity"] = mp->get_resp_addr_pool_size();
             d["states_dev"] = (uintptr_t)mp->get_doorbells_device();
             d["pool_size"] = pool->get_pool_size();
             return d;
           })
      // Writes a fragment list straight into a remote slot's descriptor block and marks the slot RX_DESCRIBED (tests of
      // the serving side's checks; the server's own describe engine never produces a list that fails them).
      .def("remote_describe_raw",
           [](ServerHolder& s, int remote_idx, int slot, std::vector<std::tuple<uint32_t, uint64_t, uint32_t>> frags) {
             P2pRpcAppRrPool* pool = s.remotes.at((size_t)remote_idx)->pool();
             P2pRpcAppRrMemPool* mp = pool->rr_mem_pool;
             if (frags.size() > mp->desc_per_slot()) throw std::invalid_argument("more fragments than the descriptor block holds");
             SrpcSlotDesc* d = mp->get_slot_desc(slot);
             uint32_t dst = 0;
             for (size_t i = 0; i < frags.size(); i++) {
               d->frag[i] = SrpcFragDesc{((uint64_t)std::get<0>(frags[i]) << 56) | std::get<1>(frags[i]), std::get<2>(frags[i]), dst};
               dst += std::get<2>(frags[i]);
             }
             d->n_frags = (uint32_t)frags.size();
             __atomic_store_n(pool->get_app_rr(slot)->h_state, (uint32_t)APP_RR_STATUS::RX_DESCRIBED, __ATOMIC_RELEASE);
           })
      .def("remote_slot_state", [](ServerHolder& s, int remote_idx, int slot) {
        return (uint32_t)__atomic_load_n(s.remotes.at((size_t)remote_idx)->pool()->get_app_rr(slot)->h_state, __ATOMIC_ACQUIRE);
      })
      .def("remote_set_slot_state", [](ServerHolder& s, int remote_idx, int slot, uint32_t v) {
        __atomic_store_n(s.remotes.at((size_t)remote_idx)->pool()->get_app_rr(slot)->h_state, v, __ATOMIC_RELEASE);
      })
      .def("remote_set_tx_off", [](ServerHolder& s, int remote_idx, int slot, uint64_t off) {
        __atomic_store_n(s.remotes.at((size_t)remote_idx)->pool()->get_app_rr(slot)->h_tx_off, off, __ATOMIC_RELEASE);
      })
      .def("remote_info",
           [](ServerHolder& s, int remote_idx) {
             const buf_mon_rr& i = s.remotes.at((size_t)remote_idx)->info();
             py::dict d;
             d["queue_size"] = i.queue_size;
             d["req_size"] = i.req_size;
             d["resp_size"] = i.resp_size;
             d["device_id"] = i.device_id;
             d["server_mode"] = i.server_mode;
             d["max_batch"] = i.max_batch;
             d["device_completes"] = i.device_completes;
             d["transform_kind"] = i.transform.kind;
             d["pull"] = i.pull;
             d["timer_offset_ns"] = i.timer_offset_ns;
             d["stamp_skew_ns"] = s.remotes.at((size_t)remote_idx)->stamp_skew_ns();
             return d;
           })
      // Sends RELEASE to every remote replica (their servers stop their workers and listen again).
      .def("release_remotes",
           [](ServerHolder& s) {
             py::gil_scoped_release rel;
             int ok = 0;
             for (auto& r : s.remotes) ok += r->release() ? 1 : 0;
             return ok;
           })
      .def("start", [](ServerHolder& s) { s.server->start(); })
      .def("stop", [](ServerHolder& s) {
        py::gil_scoped_release rel;
        s.server->stop();
      })
      .def("mark_replica_down", [](ServerHolder& s, int i, bool d) { s.server->mark_replica_down(i, d); })
      .def("stats",
           [](ServerHolder& s) {
             ServerStats st = s.server->stats();
             py::dict d;
             d["rx_pkts"] = st.rx_pkts;
             d["rx_reqs"] = st.rx_reqs;
             d["tx_resps"] = st.tx_resps;
             d["tx_pkts"] = st.tx_pkts;
             d["dropped_pkts"] = st.dropped_pkts;
             d["expired"] = st.expired;
             d["ring_full"] = st.ring_full;
             d["tx_alloc_fail"] = st.tx_alloc_fail;
             d["sg_errors"] = st.sg_errors;
             d["replicas_lost"] = st.replicas_lost;
             py::list reps;
             for (auto& r : st.replicas) {
               py::dict rd;
               rd["steered"] = r.steered;
               rd["completed"] = r.completed;
               rd["ring_full"] = r.ring_full;
               rd["pushed"] = r.pushed;
               reps.append(rd);
             }
             d["replicas"] = reps;
             return d;
           })
      // Device-timed latency samples (ns): doorbell rung by the gather -> response stored by the serving side.
      .def("device_latency_ns", [](ServerHolder& s) { return s.server->device_latency_ns(); })
      .def("clear_device_latency", [](ServerHolder& s) { s.server->clear_device_latency(); })
      .def("worker_stats", [](ServerHolder& s, int replica) {
        WorkerStats w = s.server->worker_stats(replica);
        py::dict d;
        d["num_req"] = w.num_req;
        d["num_batches"] = w.num_batches;
        d["wait_timeouts"] = w.wait_timeouts;
        d["batch_hist"] = w.batch_hist;
        d["work_ns"] = w.work_ns;
        return d;
      });

  // ---- batched server: serves one app to a producer in another process (see nvl_batched_server.h)
  py::class_<BatchedServerHolder, std::shared_ptr<BatchedServerHolder>>(m, "BatchedServer")
      .def(py::init([](std::shared_ptr<AppHolder> app, const std::string& path, uint32_t func_id, int server_mode, int max_batch) {
             auto h = std::make_shared<BatchedServerHolder>();
             if (!app->info->app_rr_pool->rr_mem_pool->exportable())
               throw std::runtime_error("BatchedServer: this app's rings cannot be shared with another process");
             h->app = app;
             h->server.reset(new NvlBatchedServer(app->info.get(), path, func_id, server_mode, max_batch));
             h->server->set_pull_engine(app->engine.get());  // a producer may ask this side to fetch requests itself
             return h;
           }),
           py::arg("app"), py::arg("path"), py::arg("func_id") = 1234, py::arg("server_mode") = 2, py::arg("max_batch") = 1)
      .def("set_ingress_stem_s2d",
           [](BatchedServerHolder& b, std::vector<float> mean, std::vector<float> inv_std) {
             if (mean.size() != 3 || inv_std.size() != 3) throw std::invalid_argument("mean / inv_std need 3 values");
             float p[6] = {mean[0], mean[1], mean[2], inv_std[0], inv_std[1], inv_std[2]};
             b.server->set_ingress_transform(SG_TRANSFORM_STEM_S2D, p);
             // and on this side's own engine, which does the gathers when the producer only describes requests
             auto* mp = b.app->info->app_rr_pool->rr_mem_pool;
             b.app->engine->set_gather_transform(SG_TRANSFORM_STEM_S2D, (uint64_t)(uintptr_t)mp->get_req_addr_range(),
                                                 (uint32_t)b.app->info->req_size, p);
           })
      .def_property_readonly("pulling", [](BatchedServerHolder& b) { return b.server->pulling(); })
      .def("pull_stats", [](BatchedServerHolder& b) {
        py::dict d;
        d["pulled"] = b.server->pulled();
        d["errors"] = b.server->pull_errors();
        return d;
      })
      // (base, bytes) of the producer's payload regions as this side's device addresses them (pull mode).
      .def("regions", [](BatchedServerHolder& b) {
        py::list l;
        uint64_t base = 0, bytes = 0;
        for (int i = 0; b.server->region(i, &base, &bytes); i++) l.append(py::make_tuple((uintptr_t)base, (size_t)bytes));
        return l;
      })
      .def("start", [](BatchedServerHolder& b) {
        if (!b.server->start()) throw std::runtime_error("BatchedServer: cannot listen on the control socket path");
      })
      .def("stop", [](BatchedServerHolder& b) {
        py::gil_scoped_release rel;
        b.server->stop();
      })
      .def_property_readonly("serving", [](BatchedServerHolder& b) { return b.server->serving(); })
      .def("counters", [](BatchedServerHolder& b) {
        py::dict d;
        d["allocs"] = b.server->counters.allocs.load();
        d["releases"] = b.server->counters.releases.load();
        d["peers_lost"] = b.server->counters.peers_lost.load();
        d["refused"] = b.server->counters.refused.load();
        return d;
      })
      .def("worker_stats", [](BatchedServerHolder& b) {
        WorkerStats w = b.server->worker_stats();
        py::dict d;
        d["num_req"] = w.num_req;
        d["num_batches"] = w.num_batches;
        d["wait_timeouts"] = w.wait_timeouts;
        d["batch_hist"] = w.batch_hist;
        d["work_ns"] = w.work_ns;
        return d;
      });

  // ---- client / load generator
  py::class_<ClientHolder, std::shared_ptr<ClientHolder>>(m, "Client")
      .def(py::init([](PortHolder port, size_t req_size, size_t resp_size, uint64_t total, uint64_t warmup,
                       const std::string& payload, bool verify, const std::string& exp_name, const std::string& out_dir,
                       const std::string& uri, int n_payloads, uint64_t seed, uint64_t drain_timeout_ns,
                       bool send_by_reference) {
             auto h = std::make_shared<ClientHolder>();
             ClientConfig c;
             c.req_size = req_size;
             c.resp_size = resp_size;
             c.total_requests = total;
             c.num_warmup = warmup;
             c.verify = verify;
             c.exp_name = exp_name;
             c.out_dir = out_dir;
             if (!uri.empty()) c.client_uri = uri;
             c.n_payloads = n_payloads;
             c.seed = seed;
             c.drain_timeout_ns = drain_timeout_ns;
             c.send_by_reference = send_by_reference;
             h->port = port;
             h->client.reset(new P2pRpcAppClient(port.port, c, req_cb_by_name(payload), resp_cb_by_name(payload)));
             h->client->PreProcessRequests();
             return h;
           }),
           py::arg("port"), py::arg("req_size") = 1024, py::arg("resp_size") = 1024, py::arg("total") = 100,
           py::arg("warmup") = 10, py::arg("payload") = "echo", py::arg("verify") = false,
           py::arg("exp_name") = "splitrpc", py::arg("out_dir") = ".", py::arg("uri") = "", py::arg("n_payloads") = 16,
           py::arg("seed") = 12345, py::arg("drain_timeout_ns") = 10000000000ull, py::arg("send_by_reference") = false)
      .def("run_closed_loop",
           [](ClientHolder& c, int outstanding) {
             py::gil_scoped_release rel;
             return c.client->run_closed_loop(outstanding);
           })
      .def("run_open_loop",
           [](ClientHolder& c, double rate, int cov, int threads) {
             py::gil_scoped_release rel;
             return c.client->run_open_loop(rate, cov, threads);
           },
           py::arg("rate"), py::arg("cov") = 1, py::arg("threads") = 1)
      .def("post_process", [](ClientHolder& c) { return c.client->PostProcessResponses(); })
      .def("save_stats", [](ClientHolder& c, bool raw) { return c.client->stats().saveStats({"sojournTime"}, raw); },
           py::arg("dump_raw") = false)
      .def("stats_json", [](ClientHolder& c) { return c.client->stats().to_json(); })
      .def("sojourn_ns", [](ClientHolder& c) { return c.client->stats().samples("sojournTime"); })
      .def("payload", [](ClientHolder& c, int i) {
        const auto& p = c.client->payload(i);
        return py::bytes((const char*)p.data(), p.size());
      })
      .def("response", [](ClientHolder& c, uint64_t i) {
        const auto& p = c.client->response(i);
        return py::bytes((const char*)p.data(), p.size());
      })
      .def_property_readonly("sent", [](ClientHolder& c) { return c.client->sent(); })
      .def_property_readonly("received", [](ClientHolder& c) { return c.client->received(); })
      .def_property_readonly("verify_failures", [](ClientHolder& c) { return c.client->verify_failures(); })
      .def_property_readonly("bad_tokens", [](ClientHolder& c) { return c.client->bad_tokens(); });

  // ---- the original's older public types (BufItemPool, first-generation records, socket records): exercised here so
  // that their behaviour is pinned by a test without exposing every method to Python.
  m.def("compat_selftest", [](int device) {
    py::dict d;
    // typed pool: host memory, and memory that a GPU addresses too
    uint32_t* hp = BufItemPool<uint32_t>::create_buf_item_pool(16, -1);
    d["host_pool"] = hp != nullptr && BufItemPool<uint32_t>::get_dev_ptr(hp) == hp && hp[15] == 0;
    BufItemPool<uint32_t>::delete_buf_item_pool(hp);
    d["host_pool_forgotten"] = BufItemPool<uint32_t>::get_dev_ptr(hp) == nullptr;
    if (device >= 0) {
      g_params* gp = BufItemPool<g_params>::create_buf_item_pool(4, device);
      d["mapped_pool"] = gp != nullptr && BufItemPool<g_params>::get_dev_ptr(gp) != nullptr;
      if (gp) BufItemPool<g_params>::delete_buf_item_pool(gp, device);
    }
    // helper names of the original
    {
      const uint64_t abs_ns = getAbsCurNs();
      d["helper_names"] = get_rpc_mtu() == rpc_mtu() && is_zerocopy_mode() == (int16_t)get_zerocopy_mode() && !getBasePath().empty() &&
                          !getDatasetBasePath().empty() && abs_ns > 1600000000ull * 1000000000ull && getCurTsAsString().size() >= 19;
      P2pRpcAppRrPool slots(4, -1, 64, 32);
      P2pRpcAppRr* r = slots.get_next();
      r->set_dummy_input_on_gpu();
      r->set_dummy_output_on_gpu();
      uint32_t in0 = 0, out0 = 7;
      std::memcpy(&in0, r->h_stub->req + 60, 4);
      std::memcpy(&out0, r->h_stub->resp + 28, 4);
      d["slot_dummy_fill"] = in0 == 1u && out0 == 0u && slots.rr_mem_pool->get_state_addr_range() == (void*)slots.rr_mem_pool->get_doorbells_host();
      P2pRpcRRPool pool(4);
      pool.setup_and_init_rr_pool(nullptr, 128);
      P2pRpcRr* any = nullptr;
      d["rr_pool_names"] = pool.get_rr_pool_container().size() == 4 && pool.get_pool_size() == 4 && pool.consume_rx_ready_rr() == nullptr &&
                           pool.consume_tx_ready_rr() == nullptr && pool.get_next_rx_ready_rr(&any) == 0;
    }
    // first-generation record + pool
    p2p_rpc_conn_info* conn = initialize_src_conn_info("b8:ce:f6:cc:6a:52,192.168.25.1,50051");
    {
      p2p_rpc_v1::P2pRpcRRPool pool(8);
      pool.setup_and_init_rr_pool(conn, 256, 64, -1);
      p2p_rpc_hdr h{};
      h.req_token = 99;
      p2p_rpc_rr* a = pool.get_rr(&h);
      p2p_rpc_rr* b = pool.get_rr(&h);
      rr_merge_req_mbuf(a, 1, 2, 3, 100, 1);
      rr_merge_req_mbuf(a, 4, 5, 6, 156, 0);
      d["v1_same_token_same_rr"] = a != nullptr && a == b;
      d["v1_merge"] = a->payload_bufs->num_items == 2 && a->req_size == 256 && a->payload_bufs->burst_items[1] == 3 &&
                      a->payload_bufs->item_size[0] == 156 && a->req_payload != nullptr && a->max_resp_size == 64;
      p2p_rpc_rr* c = rr_clone_alloc(a);
      d["v1_clone"] = c->max_req_size == 256 && c->payload_bufs->num_items == 0;
      rr_base_free(c);
      pool.reap_rr(a);
      d["v1_reaped"] = pool.num_free() == 8 && a->req_size == 0 && a->payload_bufs->num_items == 0;
      int taken = 0;
      while (pool.consume_rr()) taken++;
      d["v1_exhausts"] = taken == 8 && pool.consume_rr() == nullptr;
    }
    // first-generation synchronous app server: 32 records through two instances of the CPU echo app
    {
      CpuAppState st;
      st.req_size = st.resp_size = 64;
      p2p_rpc_v1::P2pRpcAppServer srv(cpu_app_noop, cpu_echo_run, nullptr, cpu_app_noop, 2, -1, 64, 64, 64, &st);
      p2p_rpc_v1::P2pRpcAppServer::Ring cq(64);
      srv.register_cq(&cq);
      std::vector<std::vector<uint8_t>> reqs(32, std::vector<uint8_t>(64)), resps(32, std::vector<uint8_t>(64));
      std::vector<p2p_rpc_rr*> rrs;
      for (int i = 0; i < 32; i++) {
        for (int j = 0; j < 64; j++) reqs[i][j] = (uint8_t)(i * 7 + j);
        p2p_rpc_rr* rr = rr_proto_alloc(conn, 64, 64);
        rr->req_token = 100 + i;
        rr->req_payload = reqs[i].data();
        rr->resp_payload = resps[i].data();
        rrs.push_back(rr);
      }
      srv.start();
      bool queued = true;
      for (p2p_rpc_rr* rr : rrs) queued = queued && srv.enqueue_work(rr);
      int done = 0;
      uint64_t seen = 0, t0 = getCurNs();
      p2p_rpc_rr* out = nullptr;
      while (done < 32 && getCurNs() - t0 < 5000000000ull) {
        if (cq.pop(out)) {
          done++;
          seen += out->req_token;
        } else {
          std::this_thread::yield();
        }
      }
      srv.stop();
      bool same = true;
      for (int i = 0; i < 32; i++) same = same && reqs[i] == resps[i];
      d["v1_app_server"] = srv.init_ok() && queued && done == 32 && same && srv.num_serviced() == 32 && srv.num_failed() == 0 &&
                           seen == 32 * 100 + 31 * 32 / 2;
      for (p2p_rpc_rr* rr : rrs) rr_base_free(rr);
    }
    release_conn_info(conn);
    // socket record + pool: a 2500-byte request through datagram buffers and back
    {
      size_t old_mtu = rpc_mtu();
      set_rpc_mtu(1024);
      UdpRrPool pool(4);
      pool.setup_and_init_rr_pool(2500, 40);
      UdpRpcHdr uh{};
      uh.req_token = 7;
      UdpRr* rr = pool.get_rr(&uh);
      for (size_t i = 0; i < 2500; i++) rr->req_payload[i] = (uint8_t)(i * 13);
      rr->alloc_req_bufs();
      size_t put = rr->req_to_bufs();
      const UdpRpcHdr* first = (const UdpRpcHdr*)rr->req_bufs->burst_items[0];
      const UdpRpcHdr* last = (const UdpRpcHdr*)rr->req_bufs->burst_items[2];
      d["udp_fragments"] = rr->req_bufs->num_items == 3 && put == 2500 && first->req_token == 7 && last->seq_num == 2 &&
                           rr->req_bufs->item_size[2] == UDP_RPC_HEADER_LEN + 452;
      std::vector<uint8_t> keep(rr->req_payload, rr->req_payload + 2500);
      std::memset(rr->req_payload, 0, 2500);
      size_t got = rr->bufs_to_req();
      d["udp_roundtrip"] = got == 2500 && std::memcmp(keep.data(), rr->req_payload, 2500) == 0;
      // reassembly bookkeeping by sequence number
      UdpRr other(2500, 40);
      other.rr_merge_req_buf(rr->req_bufs->burst_items[2], rr->req_bufs->item_size[2], 2);
      other.rr_merge_req_buf(rr->req_bufs->burst_items[0], rr->req_bufs->item_size[0], 0);
      bool before = other.is_req_ready();
      other.rr_merge_req_buf(rr->req_bufs->burst_items[1], rr->req_bufs->item_size[1], 1);
      d["udp_ready"] = !before && other.is_req_ready();
      other.req_bufs->num_items = 0;  // the buffers belong to rr
      pool.mark_process_rr(rr);
      UdpRr* nx = nullptr;
      d["udp_queues"] = pool.get_next_rx_ready_rr(&nx) == 1 && nx == rr && pool.consume_process_rr() == nullptr;
      pool.mark_ready_rr(rr);
      d["udp_ready_queue"] = pool.consume_ready_rr() == rr;
      pool.reap_rr(rr);
      int taken = 0;
      while (pool.consume_rr()) taken++;
      d["udp_exhausts"] = taken == 4;
      set_rpc_mtu(old_mtu);
    }
    // socket helpers of the kernel-UDP path: a 2500-byte request and a 40-byte response between two sockets
    {
      size_t old_mtu = rpc_mtu();
      set_rpc_mtu(1024);
      sockaddr_in a_srv{}, a_cli{};
      a_srv.sin_family = a_cli.sin_family = AF_INET;
      inet_pton(AF_INET, "127.0.0.1", &a_srv.sin_addr);
      inet_pton(AF_INET, "127.0.0.1", &a_cli.sin_addr);
      int s_srv = initUdpSock(&a_srv), s_cli = initUdpSock(&a_cli);
      socklen_t sl = sizeof(a_srv);
      getsockname(s_srv, (sockaddr*)&a_srv, &sl);
      bool ok = s_srv >= 0 && s_cli >= 0;
      UdpRrPool srv_pool(4), cli_pool(4);
      srv_pool.setup_and_init_rr_pool(2500, 40);
      cli_pool.setup_and_init_rr_pool(2500, 40);
      UdpRpcHdr uh{};
      uh.req_token = 4242;
      UdpRr* call = cli_pool.get_rr(&uh);
      seedGenerator(7);
      for (size_t i = 0; i < 2500; i++) call->req_payload[i] = (uint8_t)uniformint(0, 255);
      call->si_other = a_srv;
      call->alloc_req_bufs();
      call->req_to_bufs();
      ok = ok && udp_rr_send_req(s_cli, call) >= 0;
      UdpRr* got = nullptr;
      for (int tries = 0; ok && !got && tries < 50; tries++) udp_rr_recv_req(s_srv, &got, &srv_pool);
      ok = ok && got != nullptr && got->req_token == 4242;
      if (ok) {
        got->bufs_to_req();
        ok = std::memcmp(got->req_payload, call->req_payload, 2500) == 0;
        for (size_t i = 0; i < 40; i++) got->resp_payload[i] = (uint8_t)(i * 3);
        got->alloc_resp_bufs();
        got->resp_to_bufs();
        ok = ok && udp_rr_send_resp(s_srv, got) >= 0;
        UdpRr* back = nullptr;
        for (int tries = 0; ok && !back && tries < 50; tries++) udp_rr_recv_resp(s_cli, &back, &cli_pool);
        ok = ok && back == call;
        if (ok) {
          back->bufs_to_resp();
          for (size_t i = 0; i < 40; i++) ok = ok && back->resp_payload[i] == (uint8_t)(i * 3);
        }
      }
      d["udp_socket_helpers"] = ok;
      if (s_srv >= 0) ::close(s_srv);
      if (s_cli >= 0) ::close(s_cli);
      set_rpc_mtu(old_mtu);
    }
    return d;
  }, py::arg("device") = -1);

  // ---- arrival processes
  m.def("arrival_schedule", [](double rate, int cov, uint64_t n, uint64_t seed) {
    LoadGenerator lg(1.0 / rate, cov, seed);
    std::vector<uint64_t> t(n);
    uint64_t cur = 0;
    for (auto& x : t) x = cur = lg.nextReqArr(cur, false);
    return t;
  });

  // ---- model files in the original's formats
  m.def("load_lenet_ref_weights", [](const std::string& dataset_dir) {
    std::vector<std::vector<float>> w;
    if (!load_lenet_ref_weights(dataset_dir, &w)) throw std::runtime_error("cannot read data/lenet/data{2,0,1,3}.dat under " + dataset_dir);
    std::vector<py::array_t<float>> out;
    for (auto& v : w) out.emplace_back(py::array_t<float>((ssize_t)v.size(), v.data()));
    return out;
  });
  m.def("load_lstm_constants", [](const std::string& dir, const std::string& manifest, int layers, int H) {
    std::vector<std::vector<float>> w;
    std::string err = load_lstm_constant_dir(dir, manifest, layers, H, &w);
    if (!err.empty()) throw std::runtime_error("load_lstm_constants: " + err);
    std::vector<py::array_t<float>> out;
    for (auto& v : w) out.emplace_back(py::array_t<float>((ssize_t)v.size(), v.data()));
    return out;
  }, py::arg("dir"), py::arg("manifest"), py::arg("layers") = 8, py::arg("H") = 256);

  // ---- CPU oracles callable on numpy arrays
  m.def("cpu_lenet5", [](const std::vector<py::array_t<float, py::array::c_style | py::array::forcecast>>& weights,
                         py::array_t<float, py::array::c_style | py::array::forcecast> x) {
    CpuAppState s;
    s.weights = to_weights(weights);
    ssize_t n = x.size() / 784;
    py::array_t<float> out({n, (ssize_t)10});
    for (ssize_t i = 0; i < n; i++) cpu_lenet5_one(&s, x.data() + i * 784, out.mutable_data() + i * 10);
    return out;
  });
  m.def("cpu_lstm", [](const std::vector<py::array_t<float, py::array::c_style | py::array::forcecast>>& weights,
                       py::array_t<float, py::array::c_style | py::array::forcecast> x, int layers, int steps, int H) {
    auto w = to_weights(weights);
    py::array_t<float> out((ssize_t)H);
    cpu_lstm_forward(w, layers, steps, H, 0.0f, x.data(), out.mutable_data());
    return out;
  });

  bind_ops(m);
}

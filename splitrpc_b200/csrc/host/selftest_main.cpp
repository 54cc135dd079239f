// Stand-alone exercise of the host core (no Python, no CUDA) for sanitizer builds:
//
//   g++ -std=c++17 -O1 -g -fsanitize=thread            -pthread -I splitrpc_b200/csrc selftest_main.cpp -o selftest_tsan
//   g++ -std=c++17 -O1 -g -fsanitize=address,undefined -pthread -I splitrpc_b200/csrc selftest_main.cpp -o selftest_asan
//
// It runs the real server threads (receive, shunter, workers), the CPU scatter-gather engine, CPU apps, the load
// generator with host-side fault injection, and replicas behind batched servers reached over the control socket
// (ALLOC handshake, rings and doorbells shared through memfds, responses pushed by the serving side, requests pushed
// by the ingress or fetched by the serving side from shared payload regions), all in one
// process, and exits non-zero when a reply is wrong or missing.  The original has no such harness; its host code is
// only ever run on the full testbed.
#include <algorithm>
#include <cstdio>
#include <string>

#include "host/apps_cpu.h"
#include "host/copy_path_runner.h"
#include "host/loadgen.h"
#include "host/loadgen_compat.h"
#include "host/p2p_rpc_compat.h"
#include "host/splitrpc_server.h"
#include "host/transport_rr_api.h"

// The CUDA half is absent from this build.
extern "C" const SrpcDeviceOps* srpc_cuda_ops() { return nullptr; }
extern "C" P2pRpcSgEngine* srpc_make_gpu_sg_engine(int, int) { return nullptr; }

namespace {

struct Link {
  std::unique_ptr<LoopbackPort> server, client;
};

ArenaMem shm_arena(size_t bytes) {
  auto* sm = new SrpcSharedMem;
  if (!srpc_shm_create(bytes, false, sm)) std::abort();
  ArenaMem m;
  m.host = m.dev = (uint8_t*)sm->host;
  m.bytes = bytes;
  m.fd = sm->fd;
  m.release = [sm] {
    srpc_shm_free(sm);
    delete sm;
  };
  return m;
}

Link make_link(size_t slot, size_t n) {
  Link l;
  l.server.reset(new LoopbackPort(shm_arena(slot * n), shm_arena(slot * n), slot));
  l.client.reset(new LoopbackPort(make_malloc_arena(slot * n), make_malloc_arena(slot * n), slot));
  LoopbackPort::connect(l.server.get(), l.client.get());
  return l;
}

std::unique_ptr<P2pRpcAppInfo> make_cpu_app(AppRunCB run, size_t req, size_t resp, int pool, int batch) {
  auto* st = new CpuAppState;
  st->req_size = req;
  st->resp_size = resp;
  return std::unique_ptr<P2pRpcAppInfo>(new P2pRpcAppInfo(cpu_app_noop, run, [](AppCtx* c) {
    delete cpu_state(c);
    c->app_ctx_internal = nullptr;
    return 1;
  }, cpu_app_noop, -1, req, resp, pool, st, 1, batch));
}

int fails = 0;
void expect(bool ok, const char* what) {
  std::printf("%s  %s\n", ok ? "ok  " : "FAIL", what);
  if (!ok) fails++;
}

// Echo through every worker mode, with duplicated and reordered fragments on the wire.
void scenario_modes() {
  set_rpc_mtu(1024);
  for (int mode = 0; mode < 3; mode++) {
    Link l = make_link(1024, 2048);
    LoopbackFaults f;
    f.duplicate = 0.05;
    f.reorder = 0.2;
    f.seed = 7;
    l.client->set_faults(f);
    auto app = make_cpu_app(cpu_echo_run, 4096, 1024, 64, mode == 2 ? 4 : 1);
    P2pRpcSgCpuEngine engine;
    ServerConfig sc;
    sc.req_size = 4096;
    sc.resp_size = 1024;
    sc.server_mode = mode;
    sc.max_batch = mode == 2 ? 4 : 1;
    SplitRpcServer srv(l.server.get(), sc);
    srv.add_replica(app.get(), &engine);
    srv.start();
    ClientConfig cc;
    cc.req_size = 4096;
    cc.resp_size = 1024;
    cc.total_requests = 300;
    cc.num_warmup = 0;
    cc.verify = true;
    P2pRpcAppClient cli(l.client.get(), cc, echo_fill, echo_check);
    cli.PreProcessRequests();
    bool ok = cli.run_closed_loop(6);
    srv.stop();
    expect(ok && cli.received() == 300 && cli.verify_failures() == 0, mode == 0 ? "echo, sync worker" : (mode == 1 ? "echo, armed worker" : "echo, dynamic batching"));
  }
}

// One local replica plus one replica behind a batched server (control socket, shared rings), least-outstanding steering.
void scenario_remote(const std::string& sock) {
  set_rpc_mtu(1024);
  auto remote_app = make_cpu_app(cpu_vec_add_run, 2048, 1024, 64, 4);
  NvlBatchedServer bs(remote_app.get(), sock, 55, 2, 4);
  expect(bs.start(), "batched server listens");
  Link l = make_link(1024, 2048);
  auto local_app = make_cpu_app(cpu_vec_add_run, 2048, 1024, 64, 4);
  P2pRpcSgCpuEngine engine;
  ServerConfig sc;
  sc.req_size = 2048;
  sc.resp_size = 1024;
  sc.server_mode = 2;
  sc.max_batch = 4;
  sc.steer_policy = 1;
  {
    SplitRpcServer srv(l.server.get(), sc);
    srv.add_replica(local_app.get(), &engine);
    std::string err;
    auto remote = NvlRemoteReplica::connect(sock, 55, -1, 2, srv.tx_arena(), 3000, &err);
    expect(remote != nullptr, "ALLOC handshake");
    if (!remote) return;
    srv.add_remote_replica(remote.get());
    srv.start();
    ClientConfig cc;
    cc.req_size = 2048;
    cc.resp_size = 1024;
    cc.total_requests = 400;
    cc.num_warmup = 0;
    cc.verify = true;
    P2pRpcAppClient cli(l.client.get(), cc, vec_add_fill, vec_add_check);
    cli.PreProcessRequests();
    bool ok = cli.run_closed_loop(12);
    ServerStats st = srv.stats();
    srv.stop();
    expect(ok && cli.received() == 400 && cli.verify_failures() == 0, "vec_add over a local and a remote replica");
    expect(st.replicas.size() == 2 && st.replicas[0].steered > 0 && st.replicas[1].steered > 0, "both replicas served");
    expect(st.replicas[1].pushed == st.replicas[1].completed, "remote responses were pushed by the serving side");
    expect(remote->release(), "RELEASE");
  }
  bs.stop();
  expect(bs.counters.allocs == 1 && bs.counters.releases == 1 && bs.counters.peers_lost == 0, "batched server counters");
}

// Pull mode: the ingress shares its receive arena, describes each request in the slot's descriptor block, and the
// serving side's fetch thread moves the bytes (CPU engine) before its worker sees the slot.
void scenario_pull(const std::string& sock) {
  set_rpc_mtu(1024);
  auto remote_app = make_cpu_app(cpu_echo_run, 3000, 1000, 64, 4);
  P2pRpcSgCpuEngine fetch_engine;
  NvlBatchedServer bs(remote_app.get(), sock, 57, 2, 4);
  bs.set_pull_engine(&fetch_engine);
  expect(bs.start(), "batched server listens (pull)");
  Link l = make_link(1024, 2048);
  ServerConfig sc;
  sc.req_size = 3000;
  sc.resp_size = 1000;
  sc.server_mode = 2;
  sc.max_batch = 4;
  {
    SplitRpcServer srv(l.server.get(), sc);
    std::string err;
    auto remote = NvlRemoteReplica::connect(sock, 57, -1, 2, srv.tx_arena(), 3000, &err, l.server.get());
    expect(remote != nullptr && remote->pulls(), "ALLOC handshake with payload regions");
    if (!remote) return;
    srv.add_remote_replica(remote.get());
    srv.start();
    ClientConfig cc;
    cc.req_size = 3000;
    cc.resp_size = 1000;
    cc.total_requests = 300;
    cc.num_warmup = 0;
    cc.verify = true;
    P2pRpcAppClient cli(l.client.get(), cc, echo_fill, echo_check);
    cli.PreProcessRequests();
    bool ok = cli.run_closed_loop(6);
    ServerStats st = srv.stats();
    srv.stop();
    expect(ok && cli.received() == 300 && cli.verify_failures() == 0, "echo through a replica that fetches its requests itself");
    expect(st.replicas.size() == 1 && st.replicas[0].pushed == 300, "responses were pushed by the serving side");
    expect(bs.pulled() == 300 && bs.pull_errors() == 0, "every request was fetched from its descriptors");
    expect(remote->release(), "RELEASE (pull)");
  }
  bs.stop();
}

// A producer that vanishes without RELEASE.
void scenario_lost_peer(const std::string& sock) {
  auto app = make_cpu_app(cpu_echo_run, 1024, 1024, 64, 4);
  NvlBatchedServer bs(app.get(), sock, 56, 2, 4);
  bs.start();
  {
    std::string err;
    auto remote = NvlRemoteReplica::connect(sock, 56, -1, 2, nullptr, 3000, &err);
    expect(remote != nullptr && bs.serving(), "producer connected");
  }  // the connection closes here
  uint64_t t0 = getCurNs();
  while (bs.serving() && getCurNs() - t0 < 3000000000ull) usleep(1000);
  expect(!bs.serving() && bs.counters.peers_lost == 1, "server noticed the lost producer");
  bs.stop();
}

// The comparison system's copy path: eight caller threads block in the batching worker.
void scenario_copy_path() {
  auto app = make_cpu_app(cpu_echo_run, 512, 512, 16, 4);
  CopyPathBatcher batcher(app.get(), 4);
  std::vector<std::thread> callers;
  std::atomic<int> good{0};
  for (int t = 0; t < 8; t++)
    callers.emplace_back([&, t] {
      std::vector<uint8_t> req(512), resp(512);
      for (int i = 0; i < 50; i++) {
        for (int j = 0; j < 512; j++) req[j] = (uint8_t)(t * 31 + i * 7 + j);
        if (batcher.submit(req.data(), req.size(), resp.data()) && req == resp) good++;
      }
    });
  for (auto& c : callers) c.join();
  CopyPathTimes tm = batcher.times();
  batcher.stop();
  std::vector<uint8_t> req(512), resp(512);
  expect(good.load() == 400 && tm.requests == 400 && tm.batches >= 100 && tm.batches <= 400, "copy path: 400 requests through the batching worker");
  expect(!batcher.submit(req.data(), req.size(), resp.data()), "copy path: refused after stop");
}

// A serve loop written against the original's record-level transport calls (one request at a time): receive a
// complete request, flatten it, give the received packets back, take transmit buffers, write the reply (the request's
// first bytes, each plus one), set the headers from the caller's connection, send.
void scenario_record_api() {
  set_rpc_mtu(1024);
  Link l = make_link(1024, 2048);
  const size_t req = 2500, resp = 1500;
  p2p_rpc_conn_info* server_conn = initialize_src_conn_info("b8:ce:f6:cc:6a:52,192.168.25.1,50051");
  P2pRpcRRPool pool(63);
  pool.setup_and_init_rr_pool(server_conn, req);
  std::atomic<bool> cancel{false};
  std::atomic<int> served{0};
  Transport* port = l.server.get();
  std::thread server([&] {
    std::vector<uint8_t> flat(req);
    P2pRpcRr* rr = nullptr;
    while (rr_recv_sync(port, &rr, pool, cancel)) {
      gather_payload_on_cpu(rr->payload_bufs, flat.data());
      rr_release_mbufs(port, rr);
      while (rr_alloc_mbufs(port, rr, resp) == 0 && !cancel.load()) std::this_thread::yield();
      size_t off = 0;
      for (uint16_t i = 0; i < rr->payload_bufs->num_items; i++) {
        uint8_t* dst = port->tx_host_ptr(SrpcPkt{nullptr, (uint8_t*)rr->payload_bufs->burst_items[i], 0, 0});
        for (size_t k = 0; k < rr->payload_bufs->item_size[i]; k++) dst[k] = (uint8_t)(flat[off + k] + 1);
        off += rr->payload_bufs->item_size[i];
      }
      rr_set_hdr(&rr->_client_conn_info, rr, resp);
      if (rr_send(port, rr, pool)) served++;
    }
  });
  ClientConfig cc;
  cc.req_size = req;
  cc.resp_size = resp;
  cc.total_requests = 80;
  cc.num_warmup = 0;
  cc.verify = true;
  P2pRpcAppClient cli(l.client.get(), cc, vec_add_fill, [](const uint8_t* rq, const uint8_t* rs, size_t n) { return vec_add_check(rq, rs, n); });
  cli.PreProcessRequests();
  bool ok = cli.run_closed_loop(5);
  cancel.store(true);
  server.join();
  release_conn_info(server_conn);
  expect(ok && cli.received() == 80 && cli.verify_failures() == 0 && served.load() == 80 && pool.num_partial() == 0,
         "serve loop on the original's record-level transport calls: 80 requests");
}

// A driver written against the original's client interface: setters, CreateRequest / SchedRequest per call, the
// listener on a thread of its own, PostProcessResponses into the caller's statistics object.
void scenario_base_client() {
  set_rpc_mtu(1024);
  Link l = make_link(1024, 2048);
  auto app = make_cpu_app(cpu_echo_run, 3000, 3000, 64, 4);
  P2pRpcSgCpuEngine eng;
  ServerConfig sc;
  sc.req_size = sc.resp_size = 3000;
  sc.server_mode = 2;
  sc.max_batch = 4;
  SplitRpcServer srv(l.server.get(), sc);
  srv.add_replica(app.get(), &eng);
  srv.start();
  StatsManager stats("selftest_base_client", "/tmp");
  stats.startExp();
  TransportAppClient tc(&stats, l.client.get(), "");
  BaseClient* cli = &tc;
  cli->SetMaxRequests(60);
  cli->SetWarmupRequests(10);
  cli->SetMaxPayloadSize(3000, 3000);
  cli->SetVerifyRun(1);
  cli->SetReqRespCb(echo_fill, echo_check);
  cli->SetClosedLoop();
  cli->PreProcessRequests();
  std::thread listener([cli] { cli->CompleteReqListener(); });
  int issued = 0;
  while (void* tag = cli->CreateRequest(nullptr)) {
    cli->SchedRequest(tag);
    issued++;
    // at most four calls in flight
    uint64_t t0 = getCurNs();
    while ((int)tc.received() + 4 <= issued && getCurNs() - t0 < 5000000000ull) std::this_thread::yield();
  }
  uint64_t t0 = getCurNs();
  while (tc.received() < 60 && getCurNs() - t0 < 5000000000ull) std::this_thread::yield();
  cli->exit_client();
  listener.join();
  cli->PostProcessResponses();
  stats.endExp();
  srv.stop();
  expect(issued == 60 && cli->n_r_sent == 60 && cli->n_r_recv == 60 && !cli->is_client_listening() && cli->isValidToken((void*)60) &&
             !cli->isValidToken((void*)61) && stats.getRawMeasure("sojournTime").size() == 50 && tc.engine()->verify_failures() == 0,
         "original client interface: 60 calls, 50 recorded");
}

// The helper threads that share a batch of a CPU app.
void scenario_batch_pool() {
  CpuBatchPool pool(3);
  std::vector<int> hits(64);
  bool ok = true;
  for (int round = 0; round < 300; round++) {
    const int n = 1 + round % 64;
    std::fill(hits.begin(), hits.end(), 0);
    pool.run(n, [&](int i) { hits[i] += 1 + round; });
    for (int i = 0; i < 64; i++) ok = ok && hits[i] == (i < n ? 1 + round : 0);
  }
  expect(ok, "batch pool: every index exactly once, 300 rounds");
}

// First-generation synchronous app server: records through two app instances and the completion ring.
void scenario_v1_app_server() {
  CpuAppState st;
  st.req_size = st.resp_size = 128;
  p2p_rpc_v1::P2pRpcAppServer srv(cpu_app_noop, cpu_echo_run, nullptr, cpu_app_noop, 2, -1, 128, 128, 64, &st);
  p2p_rpc_v1::P2pRpcAppServer::Ring cq(64);
  srv.register_cq(&cq);
  std::vector<std::vector<uint8_t>> reqs(48, std::vector<uint8_t>(128)), resps(48, std::vector<uint8_t>(128));
  std::vector<p2p_rpc_rr*> rrs;
  for (int i = 0; i < 48; i++) {
    for (int j = 0; j < 128; j++) reqs[i][j] = (uint8_t)(i * 5 + j);
    p2p_rpc_rr* rr = rr_proto_alloc(nullptr, 128, 128);
    rr->req_payload = reqs[i].data();
    rr->resp_payload = resps[i].data();
    rrs.push_back(rr);
  }
  srv.start();
  bool queued = true;
  for (p2p_rpc_rr* rr : rrs) queued = queued && srv.enqueue_work(rr);
  int done = 0;
  uint64_t t0 = getCurNs();
  p2p_rpc_rr* out = nullptr;
  while (done < 48 && getCurNs() - t0 < 5000000000ull) {
    if (cq.pop(out)) done++;
    else std::this_thread::yield();
  }
  srv.stop();
  bool same = true;
  for (int i = 0; i < 48; i++) same = same && reqs[i] == resps[i];
  expect(queued && done == 48 && same && srv.num_serviced() == 48, "first-generation app server: 48 records through two instances");
  for (p2p_rpc_rr* rr : rrs) rr_base_free(rr);
}

}  // namespace

int main(int argc, char** argv) {
  std::string dir = argc > 1 ? argv[1] : "/tmp";
  srpc_set_log_level(SRPC_LOG_ERROR);
  scenario_modes();
  scenario_remote(dir + "/srpc_selftest_a.sock");
  scenario_pull(dir + "/srpc_selftest_c.sock");
  scenario_lost_peer(dir + "/srpc_selftest_b.sock");
  scenario_record_api();
  scenario_base_client();
  scenario_copy_path();
  scenario_batch_pool();
  scenario_v1_app_server();
  std::printf("%s\n", fails ? "SELFTEST FAILED" : "SELFTEST OK");
  return fails ? 1 : 0;
}

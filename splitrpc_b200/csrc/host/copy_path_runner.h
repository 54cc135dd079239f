// The comparison system's data path: requests that arrive in ordinary host memory (the buffers of a general-purpose
// RPC library) are copied to the device one by one, the app runs, and the responses are copied back one by one
// (reference src/grpc_bench/lenet_rpc_bench.cc:38-63 per request, src/grpc_bench/batched_grpc_handler.h:18-328 with
// an app-worker thread that drains a queue into batches).  It exists so that the split design can be measured against
// the "copy path" on the same apps, the same GPU and the same client; nothing of the serving path uses it.
//
//   CopyPathRunner   one window of the app's own request/response ring, used from slot 0: copy in, run, copy out,
//                    with a timer per phase;
//   CopyPathBatcher  the app worker: callers block in submit(); the worker thread takes what has queued up (at most
//                    max_batch), runs it as one batch and wakes the callers.
#pragma once
#include <condition_variable>
#include <cstring>
#include <deque>
#include <mutex>
#include <thread>
#include <vector>

#include "p2p_rpc_async_app_server.h"

struct CopyPathTimes {
  uint64_t h2d_ns = 0, run_ns = 0, d2h_ns = 0, batches = 0, requests = 0;
};

class CopyPathRunner {
 public:
  explicit CopyPathRunner(P2pRpcAppInfo* app) : app_(app) {
    idx_ = srv_.register_app(app);
    app->app_rr_pool->init_pool();
    // bind every slot to its place in the rings once: slot i is the i-th request / response buffer from the start
    for (int i = 0; i < app->app_rr_pool->get_pool_size(); i++) app->app_rr_pool->get_next();
  }
  int max_batch() const { return app_->app_rr_pool->get_pool_size(); }
  size_t req_size() const { return app_->app_rr_pool->req_size; }
  size_t resp_size() const { return app_->app_rr_pool->resp_size; }
  const CopyPathTimes& times() const { return t_; }

  // reqs[i] -> slot i (shorter requests are zero-padded, longer ones cut), one app run over the n slots, slot i ->
  // resps[i] (resp_size bytes each).  False when a bounded wait of the app ran out or a copy failed.
  bool run(const void* const* reqs, const size_t* lens, void* const* resps, int n) {
    if (n <= 0 || n > max_batch()) return false;
    P2pRpcAppRrPool* pool = app_->app_rr_pool;
    AppCtx* c = app_->app_ctx;
    const bool gpu = c->device_id >= 0;
    const SrpcDeviceOps* ops = gpu ? srpc_require_cuda("the copy path of a GPU app") : nullptr;
    if (gpu) ops->set_device(c->device_id);
    const size_t rq = req_size(), rs = resp_size();
    bool ok = true;
    uint64_t t0 = getCurNs();
    for (int i = 0; i < n; i++) {
      uint8_t* dst = pool->get_app_rr(i)->h_stub->req;
      const size_t len = lens[i] < rq ? lens[i] : rq;
      if (gpu) {
        ok = ok && ops->memcpy_async(dst, reqs[i], len, c->work_stream) == 0;
        if (len < rq) ok = ok && ops->memset_async(dst + len, 0, rq - len, c->work_stream) == 0;
      } else {
        std::memcpy(dst, reqs[i], len);
        if (len < rq) std::memset(dst + len, 0, rq - len);
      }
    }
    if (gpu) ok = ok && ops->stream_sync(c->work_stream) == 0;  // the original waits for the copy before it launches
    uint64_t t1 = getCurNs();
    app_->consumer_seq = 0;
    ok = ok && srv_.do_batch_work_sync(idx_, 0, n);
    uint64_t t2 = getCurNs();
    for (int i = 0; i < n; i++) {
      const uint8_t* src = pool->get_app_rr(i)->h_stub->resp;
      if (gpu) ok = ok && ops->memcpy_async(resps[i], src, rs, c->work_stream) == 0;
      else std::memcpy(resps[i], src, rs);
    }
    if (gpu) ok = ok && ops->stream_sync(c->work_stream) == 0;
    uint64_t t3 = getCurNs();
    t_.h2d_ns += t1 - t0;
    t_.run_ns += t2 - t1;
    t_.d2h_ns += t3 - t2;
    t_.batches++;
    t_.requests += (uint64_t)n;
    return ok;
  }

 private:
  P2pRpcAppInfo* app_;
  P2pRpcAsyncAppServer srv_;
  int idx_ = 0;
  CopyPathTimes t_;
};

class CopyPathBatcher {
 public:
  CopyPathBatcher(P2pRpcAppInfo* app, int max_batch) : runner_(app) {
    max_batch_ = max_batch < 1 ? 1 : (max_batch > runner_.max_batch() ? runner_.max_batch() : max_batch);
    worker_ = std::thread([this] { loop(); });
  }
  ~CopyPathBatcher() { stop(); }
  void stop() {
    {
      std::lock_guard<std::mutex> g(mu_);
      if (stopping_) return;
      stopping_ = true;
    }
    cv_.notify_all();
    if (worker_.joinable()) worker_.join();
  }
  size_t resp_size() const { return runner_.resp_size(); }
  int max_batch() const { return max_batch_; }
  CopyPathTimes times() {
    std::lock_guard<std::mutex> g(mu_);
    return times_;
  }

  // Blocks until the request has been through a batch.  False after stop() or when the run failed.
  bool submit(const void* req, size_t len, void* resp) {
    Item it{req, len, resp};
    std::unique_lock<std::mutex> lk(mu_);
    if (stopping_) return false;
    queue_.push_back(&it);
    cv_.notify_all();
    done_cv_.wait(lk, [&] { return it.done; });
    return it.ok;
  }

 private:
  struct Item {
    const void* req;
    size_t len;
    void* resp;
    bool done = false, ok = false;
  };
  void loop() {
    std::vector<Item*> batch;
    std::vector<const void*> reqs;
    std::vector<size_t> lens;
    std::vector<void*> resps;
    std::unique_lock<std::mutex> lk(mu_);
    for (;;) {
      cv_.wait(lk, [&] { return stopping_ || !queue_.empty(); });
      if (queue_.empty()) break;  // stopping and drained
      batch.clear();
      while (!queue_.empty() && (int)batch.size() < max_batch_) {
        batch.push_back(queue_.front());
        queue_.pop_front();
      }
      reqs.clear();
      lens.clear();
      resps.clear();
      for (Item* it : batch) {
        reqs.push_back(it->req);
        lens.push_back(it->len);
        resps.push_back(it->resp);
      }
      lk.unlock();
      const bool ok = runner_.run(reqs.data(), lens.data(), resps.data(), (int)batch.size());
      lk.lock();
      times_ = runner_.times();
      for (Item* it : batch) {
        it->ok = ok;
        it->done = true;
      }
      done_cv_.notify_all();
    }
    for (Item* it : queue_) it->done = true;
    queue_.clear();
    done_cv_.notify_all();
  }

  CopyPathRunner runner_;
  CopyPathTimes times_;
  int max_batch_ = 1;
  std::mutex mu_;
  std::condition_variable cv_, done_cv_;
  std::deque<Item*> queue_;
  bool stopping_ = false;
  std::thread worker_;
};

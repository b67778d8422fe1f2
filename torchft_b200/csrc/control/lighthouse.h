// Lighthouse: the job-wide quorum service.  Replica-group managers send heartbeats and
// blocking Quorum requests; a tick thread (and every incoming request) evaluates
// quorum_compute and publishes a new quorum to all waiting requesters.  The same port
// serves an HTML dashboard ("/", "/status", POST "/replica/<id>/kill").
// Behaviour modelled on the reference's src/lighthouse.rs:42-567.
#pragma once

#include <condition_variable>
#include <deque>
#include <memory>
#include <mutex>
#include <string>
#include <thread>

#include "net.h"
#include "quorum.h"

namespace tft {

class Lighthouse {
 public:
  explicit Lighthouse(const LighthouseOptions& opt);
  ~Lighthouse();
  // "http://<host>:<port>"
  std::string address() const;
  int port() const { return server_->port(); }
  void shutdown();

  // One evaluation of the quorum rules; publishes a quorum when one is ready.
  void tick();

 private:
  net::Status handle_quorum(const net::CallContext& ctx, const std::string& req, std::string* resp);
  net::Status handle_heartbeat(const net::CallContext& ctx, const std::string& req, std::string* resp);
  net::HttpResponse handle_http(const net::HttpRequest& req);
  std::string render_status();
  void tick_locked();

  LighthouseOptions opt_;
  std::unique_ptr<net::Server> server_;
  std::thread tick_thread_;
  std::atomic<bool> stop_{false};

  std::mutex mu_;
  std::condition_variable cv_;
  LighthouseState state_;
  // Published quorums, newest last, each tagged with a sequence number.
  std::deque<std::pair<uint64_t, wire::Quorum>> published_;
  uint64_t seq_ = 0;
  std::string last_reason_;
};

}  // namespace tft

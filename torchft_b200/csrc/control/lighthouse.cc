#include "lighthouse.h"

#include <algorithm>
#include <chrono>
#include <sstream>

#include "manager.h"

namespace tft {

namespace {

std::string html_escape(const std::string& s) {
  std::string o;
  for (char c : s) {
    switch (c) {
      case '&': o += "&amp;"; break;
      case '<': o += "&lt;"; break;
      case '>': o += "&gt;"; break;
      case '"': o += "&quot;"; break;
      default: o.push_back(c);
    }
  }
  return o;
}

std::string json_escape(const std::string& s) {
  std::string o;
  for (char c : s) {
    if (c == '"' || c == '\\') { o.push_back('\\'); o.push_back(c); }
    else if (static_cast<unsigned char>(c) < 0x20) o += " ";
    else o.push_back(c);
  }
  return o;
}

std::string url_decode(const std::string& s) {
  std::string o;
  for (size_t i = 0; i < s.size(); ++i) {
    if (s[i] == '%' && i + 2 < s.size()) {
      o.push_back(static_cast<char>(std::strtol(s.substr(i + 1, 2).c_str(), nullptr, 16)));
      i += 2;
    } else {
      o.push_back(s[i]);
    }
  }
  return o;
}

const char* kIndexHtml = R"HTML(<!doctype html>
<html>
<head>
<meta charset="utf-8">
<title>Lighthouse Dashboard - torchft_b200</title>
<style>
  body { margin: 0; font-family: monospace; background: #fafafa; }
  header { background: #1f2937; color: white; padding: 12px 16px; }
  header h1 { margin: 0; font-size: 20px; }
  main { padding: 0 16px 16px 16px; }
  .member { display: inline-block; border: 1px solid #444; padding: 10px; margin: 4px; background: white; }
  .member.recovering { background: #fde68a; }
  .heartbeat.old { color: #b91c1c; }
  button { margin-top: 6px; }
</style>
</head>
<body>
<header><h1>Lighthouse Dashboard</h1></header>
<main id="status">Loading...</main>
<script>
async function refresh() {
  try {
    const r = await fetch('/status');
    document.getElementById('status').innerHTML = await r.text();
  } catch (e) {}
}
async function killReplica(id) {
  await fetch('/replica/' + encodeURIComponent(id) + '/kill', {method: 'POST'});
  refresh();
}
refresh();
setInterval(refresh, 1000);
</script>
</body>
</html>
)HTML";

}  // namespace

Lighthouse::Lighthouse(const LighthouseOptions& opt) : opt_(opt) {
  server_ = std::make_unique<net::Server>(opt.bind);
  server_->add_method("/torchft.LighthouseService/Quorum",
                      [this](const net::CallContext& c, const std::string& r, std::string* o) {
                        return handle_quorum(c, r, o);
                      });
  server_->add_method("/torchft.LighthouseService/Heartbeat",
                      [this](const net::CallContext& c, const std::string& r, std::string* o) {
                        return handle_heartbeat(c, r, o);
                      });
  server_->set_http_handler([this](const net::HttpRequest& r) { return handle_http(r); });
  server_->start();
  tick_thread_ = std::thread([this] {
    while (!stop_.load()) {
      tick();
      std::this_thread::sleep_for(std::chrono::milliseconds(opt_.quorum_tick_ms));
    }
  });
  net::log_info("torchft_b200::lighthouse", "Lighthouse listening on: " + address());
}

Lighthouse::~Lighthouse() { shutdown(); }

void Lighthouse::shutdown() {
  if (stop_.exchange(true)) {
    if (tick_thread_.joinable()) tick_thread_.join();
    return;
  }
  {
    std::lock_guard<std::mutex> g(mu_);
    cv_.notify_all();
  }
  if (tick_thread_.joinable()) tick_thread_.join();
  server_->shutdown();
}

std::string Lighthouse::address() const {
  return "http://" + net::advertised_host(net::local_hostname()) + ":" + std::to_string(server_->port());
}

void Lighthouse::tick() {
  std::lock_guard<std::mutex> g(mu_);
  tick_locked();
}

void Lighthouse::tick_locked() {
  auto result = quorum_compute(net::Clock::now(), state_, opt_);
  if (result.second != last_reason_) {
    net::log_info("torchft_b200::lighthouse", "Next quorum status: " + result.second);
    last_reason_ = result.second;
  }
  if (!result.first) return;
  std::vector<wire::QuorumMember>& members = *result.first;
  // The id only moves when the ordered set of replica ids changes.
  bool forced = false;
  for (const auto& m : members) forced = forced || m.force_reconfigure;
  if (!state_.prev_quorum || forced || quorum_changed(members, state_.prev_quorum->participants)) {
    state_.quorum_id += 1;
    net::log_info("torchft_b200::lighthouse",
                  "Detected quorum change, bumping quorum_id to " + std::to_string(state_.quorum_id));
  }
  wire::Quorum q;
  q.quorum_id = state_.quorum_id;
  q.participants = members;
  auto wall = std::chrono::system_clock::now().time_since_epoch();
  q.created.seconds = std::chrono::duration_cast<std::chrono::seconds>(wall).count();
  q.created.nanos = static_cast<int32_t>(std::chrono::duration_cast<std::chrono::nanoseconds>(wall).count() % 1000000000LL);
  state_.prev_quorum = q;
  state_.participants.clear();
  published_.emplace_back(++seq_, q);
  while (published_.size() > 16) published_.pop_front();
  cv_.notify_all();
}

net::Status Lighthouse::handle_quorum(const net::CallContext& ctx, const std::string& req, std::string* resp) {
  wire::LighthouseQuorumRequest request = wire::LighthouseQuorumRequest::decode(req);
  const wire::QuorumMember& requester = request.requester;
  if (requester.replica_id.empty())
    return net::Status::Error(net::kInvalidArgument, "missing requester");
  net::log_debug("torchft_b200::lighthouse", "got quorum request for replica " + requester.replica_id);

  std::unique_lock<std::mutex> lk(mu_);
  auto join = [&] {
    state_.heartbeats[requester.replica_id] = net::Clock::now();  // a request implies liveness
    state_.participants[requester.replica_id] = MemberDetails{net::Clock::now(), requester};
  };
  join();
  uint64_t seen = seq_;
  tick_locked();  // react immediately instead of waiting for the next tick
  while (true) {
    for (const auto& entry : published_) {
      if (entry.first <= seen) continue;
      seen = entry.first;
      for (const auto& m : entry.second.participants) {
        if (m.replica_id == requester.replica_id) {
          wire::LighthouseQuorumResponse out;
          out.quorum = entry.second;
          *resp = out.encode();
          return net::Status::Ok();
        }
      }
      // Published without us (for instance a shrink-only round): ask again.
      join();
    }
    cv_.wait_for(lk, std::chrono::milliseconds(50));
    if (stop_.load()) return net::Status::Error(net::kUnavailable, "lighthouse shutting down");
    lk.unlock();
    const bool gone = ctx.cancelled();
    lk.lock();
    if (gone) return net::Status::Error(net::kDeadlineExceeded, "quorum request cancelled or timed out");
  }
}

net::Status Lighthouse::handle_heartbeat(const net::CallContext&, const std::string& req, std::string* resp) {
  wire::LighthouseHeartbeatRequest request = wire::LighthouseHeartbeatRequest::decode(req);
  std::lock_guard<std::mutex> g(mu_);
  state_.heartbeats[request.replica_id] = net::Clock::now();
  resp->clear();
  return net::Status::Ok();
}

std::string Lighthouse::render_status() {
  std::lock_guard<std::mutex> g(mu_);
  const auto now = net::Clock::now();
  auto next = quorum_compute(now, state_, opt_);
  std::ostringstream o;
  o << "Current quorum_id: " << state_.quorum_id << " <br>\n";
  o << "Next quorum status: " << html_escape(next.second) << "\n";
  o << "<h3>Previous Quorum</h3>\n";
  if (state_.prev_quorum) {
    const wire::Quorum& q = *state_.prev_quorum;
    int64_t max_step = -1;
    for (const auto& m : q.participants) max_step = std::max(max_step, m.step);
    auto wall = std::chrono::system_clock::now().time_since_epoch();
    double age = std::chrono::duration<double>(wall).count() -
                 (static_cast<double>(q.created.seconds) + q.created.nanos * 1e-9);
    o << "Previous quorum id: " << q.quorum_id << " <br>\n";
    o << "Num participants: " << q.participants.size() << " <br>\n";
    o << "Quorum age: " << age << "s\n<div>\n";
    for (const auto& m : q.participants) {
      o << "<div class=\"member" << (m.step != max_step ? " recovering" : "") << "\">\n";
      o << "  <b>" << html_escape(m.replica_id) << "</b> <br/>\n";
      o << "  Step: " << m.step << " <br/>\n";
      o << "  Manager: " << html_escape(m.address) << " <br/>\n";
      o << "  TCPStore: " << html_escape(m.store_address) << " <br/>\n";
      o << "  World size: " << m.world_size << " <br/>\n";
      o << "  <button onclick=\"killReplica('" << html_escape(m.replica_id) << "')\">Kill</button>\n";
      o << "</div>\n";
    }
    o << "</div>\n";
  }
  o << "<h2>Heartbeats</h2>\n<ul>\n";
  for (const auto& kv : state_.heartbeats) {
    double age = std::chrono::duration<double>(now - kv.second).count();
    bool old = now - kv.second >= std::chrono::milliseconds(opt_.heartbeat_timeout_ms);
    o << "  <li class=\"heartbeat" << (old ? " old" : "") << "\">" << html_escape(kv.first) << ": seen " << age
      << "s ago</li>\n";
  }
  o << "</ul>\n";
  return o.str();
}

net::HttpResponse Lighthouse::handle_http(const net::HttpRequest& req) {
  net::HttpResponse resp;
  if (req.method == "GET" && (req.path == "/" || req.path == "/index.html")) {
    resp.body = kIndexHtml;
    return resp;
  }
  if (req.method == "GET" && req.path == "/status") {
    resp.body = render_status();
    return resp;
  }
  if (req.method == "GET" && req.path == "/status.json") {
    std::lock_guard<std::mutex> g(mu_);
    std::ostringstream o;
    o << "{\"quorum_id\": " << state_.quorum_id << ", \"participants\": [";
    if (state_.prev_quorum) {
      bool first = true;
      for (const auto& m : state_.prev_quorum->participants) {
        o << (first ? "" : ", ") << "{\"replica_id\": \"" << json_escape(m.replica_id) << "\", \"step\": " << m.step
          << ", \"address\": \"" << json_escape(m.address) << "\", \"world_size\": " << m.world_size << "}";
        first = false;
      }
    }
    o << "], \"heartbeats\": " << state_.heartbeats.size() << "}";
    resp.content_type = "application/json";
    resp.body = o.str();
    return resp;
  }
  if (req.method == "GET" && req.path == "/metrics") {
    // Prometheus text exposition format
    std::lock_guard<std::mutex> g(mu_);
    const auto now = net::Clock::now();
    std::ostringstream o;
    o << "# HELP torchft_quorum_id Identifier of the current quorum (changes with membership).\n"
      << "# TYPE torchft_quorum_id gauge\ntorchft_quorum_id " << state_.quorum_id << "\n"
      << "# HELP torchft_quorums_published_total Quorums handed out since start.\n"
      << "# TYPE torchft_quorums_published_total counter\ntorchft_quorums_published_total " << seq_ << "\n"
      << "# HELP torchft_quorum_participants Members of the current quorum.\n"
      << "# TYPE torchft_quorum_participants gauge\ntorchft_quorum_participants "
      << (state_.prev_quorum ? state_.prev_quorum->participants.size() : 0) << "\n"
      << "# HELP torchft_waiting_participants Replica groups waiting for the next quorum.\n"
      << "# TYPE torchft_waiting_participants gauge\ntorchft_waiting_participants " << state_.participants.size() << "\n"
      << "# HELP torchft_heartbeat_age_seconds Time since the last heartbeat of a replica group.\n"
      << "# TYPE torchft_heartbeat_age_seconds gauge\n";
    for (const auto& kv : state_.heartbeats) {
      const double age = std::chrono::duration<double>(now - kv.second).count();
      o << "torchft_heartbeat_age_seconds{replica_id=\"" << json_escape(kv.first) << "\"} " << age << "\n";
    }
    if (state_.prev_quorum) {
      o << "# HELP torchft_replica_step Step reported by a member when the current quorum formed.\n"
        << "# TYPE torchft_replica_step gauge\n";
      for (const auto& m : state_.prev_quorum->participants)
        o << "torchft_replica_step{replica_id=\"" << json_escape(m.replica_id) << "\"} " << m.step << "\n";
    }
    resp.content_type = "text/plain; version=0.0.4";
    resp.body = o.str();
    return resp;
  }
  const std::string prefix = "/replica/";
  const std::string suffix = "/kill";
  if (req.method == "POST" && req.path.compare(0, prefix.size(), prefix) == 0 && req.path.size() > prefix.size() + suffix.size() &&
      req.path.compare(req.path.size() - suffix.size(), suffix.size(), suffix) == 0) {
    std::string replica_id = url_decode(req.path.substr(prefix.size(), req.path.size() - prefix.size() - suffix.size()));
    std::string addr;
    {
      std::lock_guard<std::mutex> g(mu_);
      if (state_.prev_quorum)
        for (const auto& m : state_.prev_quorum->participants)
          if (m.replica_id == replica_id) addr = m.address;
    }
    if (addr.empty()) {
      resp.status = 500;
      resp.content_type = "text/plain";
      resp.body = "Something went wrong: failed to find replica";
      return resp;
    }
    try {
      net::Client client(addr, std::chrono::seconds(10));
      wire::KillRequest kill;
      kill.msg = "killed from dashboard";
      client.call("/torchft.ManagerService/Kill", kill.encode(), net::Millis(10000));
    } catch (const net::RpcError& e) {
      // The target exits inside the handler, so a dropped connection is the expected outcome.
      if (e.code != net::kUnavailable) {
        resp.status = 500;
        resp.content_type = "text/plain";
        resp.body = std::string("Something went wrong: ") + e.what();
        return resp;
      }
    }
    resp.body = "";
    return resp;
  }
  resp.status = 404;
  resp.content_type = "text/plain";
  resp.body = "not found";
  return resp;
}

}  // namespace tft

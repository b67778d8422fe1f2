#include "manager.h"

#include <unistd.h>

#include <cstdlib>

namespace tft {

// ---------------------------------------------------------------- clients
wire::Quorum LighthouseClient::quorum(const wire::QuorumMember& requester, net::Millis timeout) {
  wire::LighthouseQuorumRequest req;
  req.requester = requester;
  std::string resp = client_.call("/torchft.LighthouseService/Quorum", req.encode(), timeout);
  return wire::LighthouseQuorumResponse::decode(resp).quorum;
}

void LighthouseClient::heartbeat(const std::string& replica_id, net::Millis timeout) {
  wire::LighthouseHeartbeatRequest req;
  req.replica_id = replica_id;
  client_.call("/torchft.LighthouseService/Heartbeat", req.encode(), timeout);
}

wire::ManagerQuorumResponse ManagerClient::quorum(int64_t rank, int64_t step, const std::string& checkpoint_metadata,
                                                  bool shrink_only, net::Millis timeout, bool force_reconfigure) {
  wire::ManagerQuorumRequest req;
  req.rank = rank;
  req.step = step;
  req.checkpoint_metadata = checkpoint_metadata;
  req.shrink_only = shrink_only;
  req.force_reconfigure = force_reconfigure;
  std::string resp = client_.call("/torchft.ManagerService/Quorum", req.encode(), timeout);
  return wire::ManagerQuorumResponse::decode(resp);
}

std::string ManagerClient::checkpoint_metadata(int64_t rank, net::Millis timeout) {
  wire::CheckpointMetadataRequest req;
  req.rank = rank;
  std::string resp = client_.call("/torchft.ManagerService/CheckpointMetadata", req.encode(), timeout);
  return wire::CheckpointMetadataResponse::decode(resp).checkpoint_metadata;
}

bool ManagerClient::should_commit(int64_t rank, int64_t step, bool should_commit, net::Millis timeout) {
  wire::ShouldCommitRequest req;
  req.rank = rank;
  req.step = step;
  req.should_commit = should_commit;
  std::string resp = client_.call("/torchft.ManagerService/ShouldCommit", req.encode(), timeout);
  return wire::ShouldCommitResponse::decode(resp).should_commit;
}

void ManagerClient::kill(const std::string& msg, net::Millis timeout) {
  wire::KillRequest req;
  req.msg = msg;
  client_.call("/torchft.ManagerService/Kill", req.encode(), timeout);
}

// ---------------------------------------------------------------- server
ManagerServer::ManagerServer(const std::string& replica_id, const std::string& lighthouse_addr,
                             const std::string& hostname, const std::string& bind, const std::string& store_addr,
                             uint64_t world_size, net::Millis heartbeat_interval, net::Millis connect_timeout)
    : replica_id_(replica_id),
      lighthouse_addr_(lighthouse_addr),
      hostname_(hostname),
      store_addr_(store_addr),
      world_size_(world_size),
      heartbeat_interval_(heartbeat_interval),
      connect_timeout_(connect_timeout) {
  server_ = std::make_unique<net::Server>(bind);
  quorum_client_ = std::make_unique<LighthouseClient>(lighthouse_addr, connect_timeout);
  server_->add_method("/torchft.ManagerService/Quorum",
                      [this](const net::CallContext& c, const std::string& r, std::string* o) {
                        return handle_quorum(c, r, o);
                      });
  server_->add_method("/torchft.ManagerService/CheckpointMetadata",
                      [this](const net::CallContext& c, const std::string& r, std::string* o) {
                        return handle_checkpoint_metadata(c, r, o);
                      });
  server_->add_method("/torchft.ManagerService/ShouldCommit",
                      [this](const net::CallContext& c, const std::string& r, std::string* o) {
                        return handle_should_commit(c, r, o);
                      });
  server_->add_method("/torchft.ManagerService/Kill",
                      [this](const net::CallContext& c, const std::string& r, std::string* o) {
                        return handle_kill(c, r, o);
                      });
  server_->start();
  net::log_info("torchft_b200::manager", "[Replica " + replica_id_ + "] Manager listening on " + address());

  heartbeat_thread_ = std::thread([this] {
    std::unique_ptr<LighthouseClient> hb;
    while (!stop_.load()) {
      try {
        if (!hb) hb = std::make_unique<LighthouseClient>(lighthouse_addr_, connect_timeout_);
        hb->heartbeat(replica_id_, std::max(net::Millis(1000), heartbeat_interval_ * 10));
      } catch (const std::exception&) {
        // Failed heartbeats are ignored: the lighthouse ages this replica out by itself.
      }
      const auto until = net::Clock::now() + heartbeat_interval_;
      while (!stop_.load() && net::Clock::now() < until)
        std::this_thread::sleep_for(std::min<net::Millis>(heartbeat_interval_, net::Millis(20)));
    }
  });
}

ManagerServer::~ManagerServer() { shutdown(); }

void ManagerServer::shutdown() {
  if (stop_.exchange(true)) {
    if (heartbeat_thread_.joinable()) heartbeat_thread_.join();
    return;
  }
  {
    std::lock_guard<std::mutex> g(mu_);
    cv_.notify_all();
  }
  if (heartbeat_thread_.joinable()) heartbeat_thread_.join();
  server_->shutdown();
}

std::string ManagerServer::address() const {
  return "http://" + net::advertised_host(hostname_) + ":" + std::to_string(server_->port());
}

net::Status ManagerServer::handle_quorum(const net::CallContext& ctx, const std::string& req, std::string* resp) {
  if (!ctx.timeout) return net::Status::Error(net::kInvalidArgument, "missing timeout");
  const net::Millis timeout = std::chrono::duration_cast<net::Millis>(*ctx.timeout);
  wire::ManagerQuorumRequest request = wire::ManagerQuorumRequest::decode(req);
  const int64_t rank = request.rank;
  net::log_debug("torchft_b200::manager",
                "[Replica " + replica_id_ + "] Start quorum for rank " + std::to_string(rank));

  std::unique_lock<std::mutex> lk(mu_);
  checkpoint_metadata_[rank] = request.checkpoint_metadata;
  participants_.insert(rank);
  round_force_reconfigure_ = round_force_reconfigure_ || request.force_reconfigure;
  const uint64_t my_seq = quorum_seq_;

  if (participants_.size() >= world_size_ && !quorum_in_flight_) {
    // Every local rank asked: this handler makes the group's lighthouse request.
    participants_.clear();
    quorum_in_flight_ = true;
    wire::QuorumMember me;
    me.replica_id = replica_id_;
    me.address = address();
    me.store_address = store_addr_;
    me.step = request.step;
    me.world_size = world_size_;
    me.shrink_only = request.shrink_only;
    me.force_reconfigure = round_force_reconfigure_;
    round_force_reconfigure_ = false;
    lk.unlock();
    net::Status st;
    wire::Quorum q;
    try {
      q = quorum_client_->quorum(me, timeout);
    } catch (const net::RpcError& e) {
      if (e.is_timeout())
        st = net::Status::Error(net::kCancelled, std::string("lighthouse quorum timed out: ") + e.what());
      else
        st = net::Status::Error(e.code, std::string("lighthouse quorum failed: ") + e.what());
    }
    lk.lock();
    quorum_in_flight_ = false;
    last_quorum_ = q;
    last_quorum_status_ = st;
    ++quorum_seq_;
    cv_.notify_all();
  } else {
    while (quorum_seq_ == my_seq) {
      cv_.wait_for(lk, std::chrono::milliseconds(50));
      if (quorum_seq_ != my_seq) break;
      if (stop_.load()) return net::Status::Error(net::kUnavailable, "manager shutting down");
      lk.unlock();
      const bool gone = ctx.cancelled();
      lk.lock();
      if (gone && quorum_seq_ == my_seq) {
        participants_.erase(rank);
        return net::Status::Error(net::kCancelled, "quorum request timed out waiting for local ranks");
      }
    }
  }
  if (!last_quorum_status_.ok()) return last_quorum_status_;
  const wire::Quorum quorum = last_quorum_;
  lk.unlock();
  try {
    wire::ManagerQuorumResponse out = compute_quorum_results(replica_id_, rank, quorum);
    if (out.heal)
      net::log_info("torchft_b200::manager",
                    "[Replica " + replica_id_ + "] healing is required max_step=" + std::to_string(out.max_step) +
                        ", recover_src_rank=" + std::to_string(*out.recover_src_rank));
    *resp = out.encode();
  } catch (const net::RpcError& e) {
    // e.what() is already "status: ..., message: ..."; rebuild the bare message
    return net::Status::Error(e.code, "replica " + replica_id_ + " not participating in returned quorum");
  }
  return net::Status::Ok();
}

net::Status ManagerServer::handle_checkpoint_metadata(const net::CallContext&, const std::string& req,
                                                      std::string* resp) {
  wire::CheckpointMetadataRequest request = wire::CheckpointMetadataRequest::decode(req);
  std::lock_guard<std::mutex> g(mu_);
  auto it = checkpoint_metadata_.find(request.rank);
  if (it == checkpoint_metadata_.end()) return net::Status::Error(net::kInvalidArgument, "rank not found");
  wire::CheckpointMetadataResponse out;
  out.checkpoint_metadata = it->second;
  *resp = out.encode();
  return net::Status::Ok();
}

net::Status ManagerServer::handle_should_commit(const net::CallContext& ctx, const std::string& req,
                                                std::string* resp) {
  wire::ShouldCommitRequest request = wire::ShouldCommitRequest::decode(req);
  std::unique_lock<std::mutex> lk(mu_);
  if (!request.should_commit) commit_failures_.insert(request.rank);
  commit_votes_.insert(request.rank);
  const uint64_t my_seq = commit_seq_;
  if (commit_votes_.size() >= world_size_) {
    last_commit_decision_ = commit_failures_.empty();
    net::log_debug("torchft_b200::manager", "[Replica " + replica_id_ + "] should_commit completed should_commit=" +
                                               (last_commit_decision_ ? "true" : "false"));
    commit_votes_.clear();
    commit_failures_.clear();
    ++commit_seq_;
    cv_.notify_all();
  } else {
    while (commit_seq_ == my_seq) {
      cv_.wait_for(lk, std::chrono::milliseconds(50));
      if (commit_seq_ != my_seq) break;
      if (stop_.load()) return net::Status::Error(net::kUnavailable, "manager shutting down");
      lk.unlock();
      const bool gone = ctx.cancelled();
      lk.lock();
      if (gone && commit_seq_ == my_seq) {
        commit_votes_.erase(request.rank);
        commit_failures_.erase(request.rank);
        return net::Status::Error(net::kCancelled, "should_commit timed out waiting for local ranks");
      }
    }
  }
  wire::ShouldCommitResponse out;
  out.should_commit = last_commit_decision_;
  *resp = out.encode();
  return net::Status::Ok();
}

net::Status ManagerServer::handle_kill(const net::CallContext&, const std::string& req, std::string*) {
  wire::KillRequest request = wire::KillRequest::decode(req);
  net::log_info("torchft_b200::manager", "[Replica " + replica_id_ + "] got kill request: " + request.msg);
  std::_Exit(1);
  return net::Status::Ok();
}

}  // namespace tft

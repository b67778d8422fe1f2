// Per-replica-group manager server and its clients.
//
// The server runs inside local rank 0 of a replica group.  It gathers the Quorum
// requests of all local ranks, makes ONE lighthouse request for the group, fans the
// answer out (each rank gets its own compute_quorum_results view), runs the
// should_commit barrier (logical AND over the ranks), serves checkpoint metadata to
// recovering peers, answers Kill, and heartbeats to the lighthouse.
// Behaviour modelled on the reference's src/manager.rs:40-355.
#pragma once

#include <condition_variable>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <string>
#include <thread>

#include "net.h"
#include "quorum.h"

namespace tft {

class LighthouseClient {
 public:
  LighthouseClient(const std::string& addr, net::Millis connect_timeout) : client_(addr, connect_timeout) {}
  wire::Quorum quorum(const wire::QuorumMember& requester, net::Millis timeout);
  void heartbeat(const std::string& replica_id, net::Millis timeout);

 private:
  net::Client client_;
};

class ManagerClient {
 public:
  ManagerClient(const std::string& addr, net::Millis connect_timeout) : client_(addr, connect_timeout) {}
  wire::ManagerQuorumResponse quorum(int64_t rank, int64_t step, const std::string& checkpoint_metadata,
                                     bool shrink_only, net::Millis timeout, bool force_reconfigure = false);
  std::string checkpoint_metadata(int64_t rank, net::Millis timeout);
  bool should_commit(int64_t rank, int64_t step, bool should_commit, net::Millis timeout);
  void kill(const std::string& msg, net::Millis timeout);

 private:
  net::Client client_;
};

class ManagerServer {
 public:
  ManagerServer(const std::string& replica_id, const std::string& lighthouse_addr, const std::string& hostname,
                const std::string& bind, const std::string& store_addr, uint64_t world_size,
                net::Millis heartbeat_interval, net::Millis connect_timeout);
  ~ManagerServer();
  std::string address() const;
  void shutdown();

 private:
  net::Status handle_quorum(const net::CallContext& ctx, const std::string& req, std::string* resp);
  net::Status handle_checkpoint_metadata(const net::CallContext& ctx, const std::string& req, std::string* resp);
  net::Status handle_should_commit(const net::CallContext& ctx, const std::string& req, std::string* resp);
  net::Status handle_kill(const net::CallContext& ctx, const std::string& req, std::string* resp);

  std::string replica_id_;
  std::string lighthouse_addr_;
  std::string hostname_;
  std::string store_addr_;
  uint64_t world_size_;
  net::Millis heartbeat_interval_;
  net::Millis connect_timeout_;

  std::unique_ptr<net::Server> server_;
  std::unique_ptr<LighthouseClient> quorum_client_;
  std::thread heartbeat_thread_;
  std::atomic<bool> stop_{false};

  std::mutex mu_;
  std::condition_variable cv_;
  // quorum round state
  std::map<int64_t, std::string> checkpoint_metadata_;
  std::set<int64_t> participants_;
  bool round_force_reconfigure_ = false;  // OR over the ranks of the current round
  uint64_t quorum_seq_ = 0;            // bumped whenever a round resolves
  bool quorum_in_flight_ = false;
  wire::Quorum last_quorum_;
  net::Status last_quorum_status_;
  // should_commit round state
  std::set<int64_t> commit_votes_;
  std::set<int64_t> commit_failures_;
  uint64_t commit_seq_ = 0;
  bool last_commit_decision_ = false;
};

}  // namespace tft

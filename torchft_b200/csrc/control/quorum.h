// Pure quorum logic of the control plane.
//
// quorum_compute decides whether the lighthouse may issue a new quorum
// (behaviour of the reference: src/lighthouse.rs:113-241);
// compute_quorum_results derives one rank's view of an issued quorum: replica rank,
// max-step cohort, rendezvous store and recovery assignments
// (behaviour of the reference: src/manager.rs:357-480).
#pragma once

#include <chrono>
#include <map>
#include <optional>
#include <string>
#include <utility>
#include <vector>

#include "net.h"
#include "wire.h"

namespace tft {

struct LighthouseOptions {
  std::string bind = "[::]:29510";
  uint64_t join_timeout_ms = 60000;
  uint64_t min_replicas = 1;
  uint64_t quorum_tick_ms = 100;
  uint64_t heartbeat_timeout_ms = 5000;
};

struct MemberDetails {
  net::Clock::time_point joined;
  wire::QuorumMember member;
};

struct LighthouseState {
  std::map<std::string, MemberDetails> participants;
  std::optional<wire::Quorum> prev_quorum;
  int64_t quorum_id = 0;
  std::map<std::string, net::Clock::time_point> heartbeats;
};

// True when the ordered lists of replica ids differ.
bool quorum_changed(const std::vector<wire::QuorumMember>& a, const std::vector<wire::QuorumMember>& b);

// Returns the members of the next quorum (sorted by replica id) if one can be issued
// now, plus a human-readable reason.
std::pair<std::optional<std::vector<wire::QuorumMember>>, std::string> quorum_compute(
    net::Clock::time_point now, const LighthouseState& state, const LighthouseOptions& opt);

// Throws net::RpcError(kNotFound) if replica_id is not part of the quorum.
wire::ManagerQuorumResponse compute_quorum_results(const std::string& replica_id, int64_t rank,
                                                   const wire::Quorum& quorum);

}  // namespace tft

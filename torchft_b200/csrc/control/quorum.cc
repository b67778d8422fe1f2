#include "quorum.h"

#include <algorithm>
#include <set>

namespace tft {

bool quorum_changed(const std::vector<wire::QuorumMember>& a, const std::vector<wire::QuorumMember>& b) {
  if (a.size() != b.size()) return true;
  for (size_t i = 0; i < a.size(); ++i)
    if (a[i].replica_id != b[i].replica_id) return true;
  return false;
}

std::pair<std::optional<std::vector<wire::QuorumMember>>, std::string> quorum_compute(
    net::Clock::time_point now, const LighthouseState& state, const LighthouseOptions& opt) {
  const auto hb_timeout = std::chrono::milliseconds(opt.heartbeat_timeout_ms);
  std::set<std::string> healthy_replicas;
  for (const auto& kv : state.heartbeats)
    if (now - kv.second < hb_timeout) healthy_replicas.insert(kv.first);

  // std::map iterates in key order, so candidates come out sorted by replica id.
  std::vector<const MemberDetails*> healthy_participants;
  for (const auto& kv : state.participants)
    if (healthy_replicas.count(kv.first)) healthy_participants.push_back(&kv.second);

  std::vector<wire::QuorumMember> candidates;
  bool shrink_only = false;
  for (const MemberDetails* d : healthy_participants) {
    candidates.push_back(d->member);
    shrink_only = shrink_only || d->member.shrink_only;
  }

  const std::string metadata = "[" + std::to_string(healthy_participants.size()) + "/" +
                               std::to_string(state.participants.size()) + " participants healthy][" +
                               std::to_string(healthy_replicas.size()) + " heartbeating][shrink_only=" +
                               (shrink_only ? "true" : "false") + "]";

  if (state.prev_quorum) {
    std::set<std::string> prev_ids;
    for (const auto& p : state.prev_quorum->participants) prev_ids.insert(p.replica_id);
    if (shrink_only) {
      std::vector<wire::QuorumMember> kept;
      for (auto& c : candidates)
        if (prev_ids.count(c.replica_id)) kept.push_back(c);
      candidates.swap(kept);
    }
    // Fast path: every member of the previous quorum asked again and is healthy.
    bool fast = true;
    for (const auto& p : state.prev_quorum->participants) {
      auto it = state.participants.find(p.replica_id);
      if (it == state.participants.end() || !healthy_replicas.count(p.replica_id)) {
        fast = false;
        break;
      }
    }
    if (fast) return {candidates, "Fast quorum found! " + metadata};
  }

  // The size rules are applied to the set that would be returned.  It differs from the healthy
  // participants only after a shrink_only filter; the reference (src/lighthouse.rs:190-213) counts the
  // unfiltered set there and can hand out a quorum below min_replicas, a minority, or an empty one.
  const size_t quorum_size = candidates.size();
  if (quorum_size < opt.min_replicas) {
    return {std::nullopt, "New quorum not ready, only have " + std::to_string(quorum_size) +
                              " participants, need min_replicas " + std::to_string(opt.min_replicas) + " " +
                              metadata};
  }

  // Split-brain guard: more than half of the replicas known to be alive must take part.
  if (quorum_size <= healthy_replicas.size() / 2) {
    return {std::nullopt, "New quorum not ready, only have " + std::to_string(quorum_size) +
                              " participants, need at least half of " +
                              std::to_string(healthy_replicas.size()) + " healthy workers " + metadata};
  }

  const bool all_joined = healthy_participants.size() == healthy_replicas.size();
  net::Clock::time_point first_joined = now;
  bool any = false;
  for (const MemberDetails* d : healthy_participants) {
    if (!any || d->joined < first_joined) first_joined = d->joined;
    any = true;
  }
  if (!all_joined && now - first_joined < std::chrono::milliseconds(opt.join_timeout_ms)) {
    return {std::nullopt,
            "Valid quorum with " + std::to_string(healthy_participants.size()) + " participants, waiting for " +
                std::to_string(healthy_replicas.size() - healthy_participants.size()) +
                " healthy but not participating stragglers due to join timeout " + metadata};
  }
  return {candidates, "Valid quorum found " + metadata};
}

wire::ManagerQuorumResponse compute_quorum_results(const std::string& replica_id, int64_t rank,
                                                   const wire::Quorum& quorum) {
  std::vector<wire::QuorumMember> members = quorum.participants;
  std::stable_sort(members.begin(), members.end(),
                   [](const wire::QuorumMember& a, const wire::QuorumMember& b) { return a.replica_id < b.replica_id; });

  int64_t replica_rank = -1;
  for (size_t i = 0; i < members.size(); ++i)
    if (members[i].replica_id == replica_id) {
      replica_rank = static_cast<int64_t>(i);
      break;
    }
  if (replica_rank < 0)
    throw net::RpcError(net::kNotFound, "replica " + replica_id + " not participating in returned quorum");

  int64_t max_step = members[0].step;
  for (const auto& m : members) max_step = std::max(max_step, m.step);
  std::vector<size_t> cohort;  // indices of the members at max_step
  for (size_t i = 0; i < members.size(); ++i)
    if (members[i].step == max_step) cohort.push_back(i);

  wire::ManagerQuorumResponse out;
  for (size_t i = 0; i < cohort.size(); ++i)
    if (members[cohort[i]].replica_id == replica_id) out.max_rank = static_cast<int64_t>(i);

  // The member whose store every rank with this local rank uses for rendezvous.
  const wire::QuorumMember& primary = members[cohort[static_cast<size_t>(rank) % cohort.size()]];

  // Behind members recover; at step 0 everyone but the primary does (initial weight sync).
  std::vector<size_t> recovering, up_to_date;
  for (size_t i = 0; i < members.size(); ++i) {
    const bool behind = members[i].step != max_step;
    const bool init = max_step == 0 && members[i].replica_id != primary.replica_id;
    (behind || init ? recovering : up_to_date).push_back(i);
  }

  // Round-robin over the up-to-date members, shifted by the local rank so that the local
  // ranks of one recovering group pull from different sources.
  for (size_t i = 0; i < recovering.size(); ++i) {
    const size_t src = up_to_date[(i + static_cast<size_t>(rank)) % up_to_date.size()];
    if (static_cast<int64_t>(src) == replica_rank) out.recover_dst_ranks.push_back(static_cast<int64_t>(recovering[i]));
    if (static_cast<int64_t>(recovering[i]) == replica_rank) out.recover_src_rank = static_cast<int64_t>(src);
  }

  out.heal = out.recover_src_rank.has_value();
  if (out.heal) out.recover_src_manager_address = members[static_cast<size_t>(*out.recover_src_rank)].address;
  out.quorum_id = quorum.quorum_id;
  out.store_address = primary.store_address;
  out.max_step = max_step;
  out.max_world_size = static_cast<int64_t>(cohort.size());
  out.replica_rank = replica_rank;
  out.replica_world_size = static_cast<int64_t>(members.size());
  return out;
}

}  // namespace tft

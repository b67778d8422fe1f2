// Protobuf wire codec for the torchft control-plane schema (package "torchft":
// QuorumMember, Quorum, Lighthouse*/Manager* requests and responses).  Field numbers and
// wire types follow the published schema so payloads are byte-compatible with any
// protobuf implementation of it; proto3 `optional` presence is tracked explicitly.
#pragma once

#include <cstdint>
#include <optional>
#include <stdexcept>
#include <string>
#include <vector>

namespace tft {
namespace wire {

struct DecodeError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

class Writer {
 public:
  void varint(uint64_t v);
  void tag(uint32_t field, uint32_t wt) { varint((uint64_t(field) << 3) | wt); }
  void put_string(uint32_t field, const std::string& s);                  // omitted if empty
  void put_bytes_always(uint32_t field, const std::string& s);            // always written
  void put_int64(uint32_t field, int64_t v);                              // omitted if 0
  void put_int64_always(uint32_t field, int64_t v);
  void put_uint64(uint32_t field, uint64_t v);
  void put_bool(uint32_t field, bool v);
  const std::string& data() const { return buf_; }
  std::string take() { return std::move(buf_); }

 private:
  std::string buf_;
};

class Reader {
 public:
  Reader(const char* p, size_t n) : p_(p), end_(p + n) {}
  explicit Reader(const std::string& s) : Reader(s.data(), s.size()) {}
  bool next(uint32_t* field, uint32_t* wt);  // false at end of buffer
  uint64_t varint();
  std::string bytes();
  void skip(uint32_t wt);

 private:
  const char* p_;
  const char* end_;
};

struct QuorumMember {
  std::string replica_id;
  std::string address;
  std::string store_address;
  int64_t step = 0;
  uint64_t world_size = 0;
  bool shrink_only = false;
  // Extension (field 7): a member whose previous step failed asks for a fresh quorum id so that
  // every member re-creates its communicator even though membership did not change.
  bool force_reconfigure = false;
  std::string encode() const;
  static QuorumMember decode(const std::string& s);
};

struct Timestamp {
  int64_t seconds = 0;
  int32_t nanos = 0;
};

struct Quorum {
  int64_t quorum_id = 0;
  std::vector<QuorumMember> participants;
  Timestamp created;
  std::string encode() const;
  static Quorum decode(const std::string& s);
};

struct LighthouseQuorumRequest {
  QuorumMember requester;
  std::string encode() const;
  static LighthouseQuorumRequest decode(const std::string& s);
};

struct LighthouseQuorumResponse {
  Quorum quorum;
  std::string encode() const;
  static LighthouseQuorumResponse decode(const std::string& s);
};

struct LighthouseHeartbeatRequest {
  std::string replica_id;
  std::string encode() const;
  static LighthouseHeartbeatRequest decode(const std::string& s);
};

struct ManagerQuorumRequest {
  int64_t rank = 0;
  int64_t step = 0;
  std::string checkpoint_metadata;
  bool shrink_only = false;
  bool force_reconfigure = false;  // extension, field 5
  std::string encode() const;
  static ManagerQuorumRequest decode(const std::string& s);
};

struct ManagerQuorumResponse {
  int64_t quorum_id = 0;
  std::string recover_src_manager_address;
  std::optional<int64_t> recover_src_rank;
  std::vector<int64_t> recover_dst_ranks;
  std::string store_address;
  int64_t max_step = 0;
  std::optional<int64_t> max_rank;
  int64_t max_world_size = 0;
  int64_t replica_rank = 0;
  int64_t replica_world_size = 0;
  bool heal = false;
  std::string encode() const;
  static ManagerQuorumResponse decode(const std::string& s);
};

struct CheckpointMetadataRequest {
  int64_t rank = 0;
  std::string encode() const;
  static CheckpointMetadataRequest decode(const std::string& s);
};

struct CheckpointMetadataResponse {
  std::string checkpoint_metadata;
  std::string encode() const;
  static CheckpointMetadataResponse decode(const std::string& s);
};

struct ShouldCommitRequest {
  bool should_commit = false;
  int64_t rank = 0;
  int64_t step = 0;
  std::string encode() const;
  static ShouldCommitRequest decode(const std::string& s);
};

struct ShouldCommitResponse {
  bool should_commit = false;
  std::string encode() const;
  static ShouldCommitResponse decode(const std::string& s);
};

struct KillRequest {
  std::string msg;
  std::string encode() const;
  static KillRequest decode(const std::string& s);
};

}  // namespace wire
}  // namespace tft

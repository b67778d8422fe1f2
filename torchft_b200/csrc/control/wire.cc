#include "wire.h"

namespace tft {
namespace wire {

namespace {
constexpr uint32_t kVarint = 0, kFixed64 = 1, kLen = 2, kFixed32 = 5;
}

void Writer::varint(uint64_t v) {
  while (v >= 0x80) {
    buf_.push_back(static_cast<char>((v & 0x7F) | 0x80));
    v >>= 7;
  }
  buf_.push_back(static_cast<char>(v));
}
void Writer::put_string(uint32_t field, const std::string& s) {
  if (s.empty()) return;
  put_bytes_always(field, s);
}
void Writer::put_bytes_always(uint32_t field, const std::string& s) {
  tag(field, kLen);
  varint(s.size());
  buf_.append(s);
}
void Writer::put_int64(uint32_t field, int64_t v) {
  if (v == 0) return;
  put_int64_always(field, v);
}
void Writer::put_int64_always(uint32_t field, int64_t v) {
  tag(field, kVarint);
  varint(static_cast<uint64_t>(v));
}
void Writer::put_uint64(uint32_t field, uint64_t v) {
  if (v == 0) return;
  tag(field, kVarint);
  varint(v);
}
void Writer::put_bool(uint32_t field, bool v) {
  if (!v) return;
  tag(field, kVarint);
  varint(1);
}

bool Reader::next(uint32_t* field, uint32_t* wt) {
  if (p_ >= end_) return false;
  uint64_t key = varint();
  *field = static_cast<uint32_t>(key >> 3);
  *wt = static_cast<uint32_t>(key & 7);
  if (*field == 0) throw DecodeError("invalid field number 0");
  return true;
}
uint64_t Reader::varint() {
  uint64_t v = 0;
  int shift = 0;
  while (true) {
    if (p_ >= end_) throw DecodeError("truncated varint");
    uint8_t b = static_cast<uint8_t>(*p_++);
    if (shift < 64) v |= static_cast<uint64_t>(b & 0x7F) << shift;
    if (!(b & 0x80)) break;
    shift += 7;
    if (shift > 70) throw DecodeError("varint too long");
  }
  return v;
}
std::string Reader::bytes() {
  uint64_t n = varint();
  if (n > static_cast<uint64_t>(end_ - p_)) throw DecodeError("truncated length-delimited field");
  std::string s(p_, p_ + n);
  p_ += n;
  return s;
}
void Reader::skip(uint32_t wt) {
  switch (wt) {
    case kVarint: varint(); break;
    case kFixed64:
      if (end_ - p_ < 8) throw DecodeError("truncated fixed64");
      p_ += 8;
      break;
    case kLen: bytes(); break;
    case kFixed32:
      if (end_ - p_ < 4) throw DecodeError("truncated fixed32");
      p_ += 4;
      break;
    default: throw DecodeError("unsupported wire type");
  }
}

// ---------------------------------------------------------------- QuorumMember
std::string QuorumMember::encode() const {
  Writer w;
  w.put_string(1, replica_id);
  w.put_string(2, address);
  w.put_string(3, store_address);
  w.put_int64(4, step);
  w.put_uint64(5, world_size);
  w.put_bool(6, shrink_only);
  w.put_bool(7, force_reconfigure);
  return w.take();
}
QuorumMember QuorumMember::decode(const std::string& s) {
  QuorumMember m;
  Reader r(s);
  uint32_t f, wt;
  while (r.next(&f, &wt)) {
    if (f == 1 && wt == kLen) m.replica_id = r.bytes();
    else if (f == 2 && wt == kLen) m.address = r.bytes();
    else if (f == 3 && wt == kLen) m.store_address = r.bytes();
    else if (f == 4 && wt == kVarint) m.step = static_cast<int64_t>(r.varint());
    else if (f == 5 && wt == kVarint) m.world_size = r.varint();
    else if (f == 6 && wt == kVarint) m.shrink_only = r.varint() != 0;
    else if (f == 7 && wt == kVarint) m.force_reconfigure = r.varint() != 0;
    else r.skip(wt);
  }
  return m;
}

// ---------------------------------------------------------------- Quorum
std::string Quorum::encode() const {
  Writer w;
  w.put_int64(1, quorum_id);
  for (const auto& p : participants) w.put_bytes_always(2, p.encode());
  if (created.seconds != 0 || created.nanos != 0) {
    Writer t;
    t.put_int64(1, created.seconds);
    t.put_int64(2, created.nanos);
    w.put_bytes_always(3, t.data());
  }
  return w.take();
}
Quorum Quorum::decode(const std::string& s) {
  Quorum q;
  Reader r(s);
  uint32_t f, wt;
  while (r.next(&f, &wt)) {
    if (f == 1 && wt == kVarint) q.quorum_id = static_cast<int64_t>(r.varint());
    else if (f == 2 && wt == kLen) q.participants.push_back(QuorumMember::decode(r.bytes()));
    else if (f == 3 && wt == kLen) {
      std::string t = r.bytes();
      Reader tr(t);
      uint32_t tf, twt;
      while (tr.next(&tf, &twt)) {
        if (tf == 1 && twt == kVarint) q.created.seconds = static_cast<int64_t>(tr.varint());
        else if (tf == 2 && twt == kVarint) q.created.nanos = static_cast<int32_t>(tr.varint());
        else tr.skip(twt);
      }
    } else r.skip(wt);
  }
  return q;
}

std::string LighthouseQuorumRequest::encode() const {
  Writer w;
  w.put_bytes_always(1, requester.encode());
  return w.take();
}
LighthouseQuorumRequest LighthouseQuorumRequest::decode(const std::string& s) {
  LighthouseQuorumRequest m;
  Reader r(s);
  uint32_t f, wt;
  while (r.next(&f, &wt)) {
    if (f == 1 && wt == kLen) m.requester = QuorumMember::decode(r.bytes());
    else r.skip(wt);
  }
  return m;
}

std::string LighthouseQuorumResponse::encode() const {
  Writer w;
  w.put_bytes_always(1, quorum.encode());
  return w.take();
}
LighthouseQuorumResponse LighthouseQuorumResponse::decode(const std::string& s) {
  LighthouseQuorumResponse m;
  Reader r(s);
  uint32_t f, wt;
  while (r.next(&f, &wt)) {
    if (f == 1 && wt == kLen) m.quorum = Quorum::decode(r.bytes());
    else r.skip(wt);
  }
  return m;
}

std::string LighthouseHeartbeatRequest::encode() const {
  Writer w;
  w.put_string(1, replica_id);
  return w.take();
}
LighthouseHeartbeatRequest LighthouseHeartbeatRequest::decode(const std::string& s) {
  LighthouseHeartbeatRequest m;
  Reader r(s);
  uint32_t f, wt;
  while (r.next(&f, &wt)) {
    if (f == 1 && wt == kLen) m.replica_id = r.bytes();
    else r.skip(wt);
  }
  return m;
}

std::string ManagerQuorumRequest::encode() const {
  Writer w;
  w.put_int64(1, rank);
  w.put_int64(2, step);
  w.put_string(3, checkpoint_metadata);
  w.put_bool(4, shrink_only);
  w.put_bool(5, force_reconfigure);
  return w.take();
}
ManagerQuorumRequest ManagerQuorumRequest::decode(const std::string& s) {
  ManagerQuorumRequest m;
  Reader r(s);
  uint32_t f, wt;
  while (r.next(&f, &wt)) {
    if (f == 1 && wt == kVarint) m.rank = static_cast<int64_t>(r.varint());
    else if (f == 2 && wt == kVarint) m.step = static_cast<int64_t>(r.varint());
    else if (f == 3 && wt == kLen) m.checkpoint_metadata = r.bytes();
    else if (f == 4 && wt == kVarint) m.shrink_only = r.varint() != 0;
    else if (f == 5 && wt == kVarint) m.force_reconfigure = r.varint() != 0;
    else r.skip(wt);
  }
  return m;
}

std::string ManagerQuorumResponse::encode() const {
  Writer w;
  w.put_int64(1, quorum_id);
  w.put_string(2, recover_src_manager_address);
  if (recover_src_rank) w.put_int64_always(3, *recover_src_rank);
  if (!recover_dst_ranks.empty()) {
    // proto3 packs repeated scalars
    Writer p;
    for (int64_t v : recover_dst_ranks) p.varint(static_cast<uint64_t>(v));
    w.put_bytes_always(4, p.data());
  }
  w.put_string(5, store_address);
  w.put_int64(6, max_step);
  if (max_rank) w.put_int64_always(7, *max_rank);
  w.put_int64(8, max_world_size);
  w.put_int64(9, replica_rank);
  w.put_int64(10, replica_world_size);
  w.put_bool(11, heal);
  return w.take();
}
ManagerQuorumResponse ManagerQuorumResponse::decode(const std::string& s) {
  ManagerQuorumResponse m;
  Reader r(s);
  uint32_t f, wt;
  while (r.next(&f, &wt)) {
    if (f == 1 && wt == kVarint) m.quorum_id = static_cast<int64_t>(r.varint());
    else if (f == 2 && wt == kLen) m.recover_src_manager_address = r.bytes();
    else if (f == 3 && wt == kVarint) m.recover_src_rank = static_cast<int64_t>(r.varint());
    else if (f == 4 && wt == kLen) {
      std::string p = r.bytes();
      const size_t n = p.size();
      size_t consumed = 0;
      while (consumed < n) {
        uint64_t v = 0;
        int shift = 0;
        while (true) {
          if (consumed >= n) throw DecodeError("truncated packed varint");
          uint8_t b = static_cast<uint8_t>(p[consumed++]);
          if (shift < 64) v |= static_cast<uint64_t>(b & 0x7F) << shift;
          if (!(b & 0x80)) break;
          shift += 7;
        }
        m.recover_dst_ranks.push_back(static_cast<int64_t>(v));
      }
    } else if (f == 4 && wt == kVarint) m.recover_dst_ranks.push_back(static_cast<int64_t>(r.varint()));
    else if (f == 5 && wt == kLen) m.store_address = r.bytes();
    else if (f == 6 && wt == kVarint) m.max_step = static_cast<int64_t>(r.varint());
    else if (f == 7 && wt == kVarint) m.max_rank = static_cast<int64_t>(r.varint());
    else if (f == 8 && wt == kVarint) m.max_world_size = static_cast<int64_t>(r.varint());
    else if (f == 9 && wt == kVarint) m.replica_rank = static_cast<int64_t>(r.varint());
    else if (f == 10 && wt == kVarint) m.replica_world_size = static_cast<int64_t>(r.varint());
    else if (f == 11 && wt == kVarint) m.heal = r.varint() != 0;
    else r.skip(wt);
  }
  return m;
}

std::string CheckpointMetadataRequest::encode() const {
  Writer w;
  w.put_int64(1, rank);
  return w.take();
}
CheckpointMetadataRequest CheckpointMetadataRequest::decode(const std::string& s) {
  CheckpointMetadataRequest m;
  Reader r(s);
  uint32_t f, wt;
  while (r.next(&f, &wt)) {
    if (f == 1 && wt == kVarint) m.rank = static_cast<int64_t>(r.varint());
    else r.skip(wt);
  }
  return m;
}

std::string CheckpointMetadataResponse::encode() const {
  Writer w;
  w.put_string(1, checkpoint_metadata);
  return w.take();
}
CheckpointMetadataResponse CheckpointMetadataResponse::decode(const std::string& s) {
  CheckpointMetadataResponse m;
  Reader r(s);
  uint32_t f, wt;
  while (r.next(&f, &wt)) {
    if (f == 1 && wt == kLen) m.checkpoint_metadata = r.bytes();
    else r.skip(wt);
  }
  return m;
}

std::string ShouldCommitRequest::encode() const {
  Writer w;
  w.put_bool(1, should_commit);
  w.put_int64(2, rank);
  w.put_int64(3, step);
  return w.take();
}
ShouldCommitRequest ShouldCommitRequest::decode(const std::string& s) {
  ShouldCommitRequest m;
  Reader r(s);
  uint32_t f, wt;
  while (r.next(&f, &wt)) {
    if (f == 1 && wt == kVarint) m.should_commit = r.varint() != 0;
    else if (f == 2 && wt == kVarint) m.rank = static_cast<int64_t>(r.varint());
    else if (f == 3 && wt == kVarint) m.step = static_cast<int64_t>(r.varint());
    else r.skip(wt);
  }
  return m;
}

std::string ShouldCommitResponse::encode() const {
  Writer w;
  w.put_bool(1, should_commit);
  return w.take();
}
ShouldCommitResponse ShouldCommitResponse::decode(const std::string& s) {
  ShouldCommitResponse m;
  Reader r(s);
  uint32_t f, wt;
  while (r.next(&f, &wt)) {
    if (f == 1 && wt == kVarint) m.should_commit = r.varint() != 0;
    else r.skip(wt);
  }
  return m;
}

std::string KillRequest::encode() const {
  Writer w;
  w.put_string(1, msg);
  return w.take();
}
KillRequest KillRequest::decode(const std::string& s) {
  KillRequest m;
  Reader r(s);
  uint32_t f, wt;
  while (r.next(&f, &wt)) {
    if (f == 1 && wt == kLen) m.msg = r.bytes();
    else r.skip(wt);
  }
  return m;
}

}  // namespace wire
}  // namespace tft

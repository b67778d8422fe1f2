#include "h2.h"

#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <algorithm>
#include <array>
#include <condition_variable>
#include <cstring>
#include <thread>

namespace tft {
namespace net {
namespace h2 {

// ================================================================ HPACK: Huffman code
//
// The code of RFC 7541 Appendix B is canonical: within one code length the codes increase with
// the symbol value, and the first code of a length continues from the last code of the shorter
// length.  So the table is fully determined by the length of each of the 257 symbols (256 =
// end of string), listed here per length.
namespace {

struct LengthGroup {
  int bits;
  std::vector<int> symbols;
};

std::vector<int> chars(const char* s) {
  std::vector<int> v;
  for (; *s; ++s) v.push_back(static_cast<unsigned char>(*s));
  return v;
}

const std::vector<LengthGroup>& length_groups() {
  static const std::vector<LengthGroup> groups = [] {
    std::vector<LengthGroup> g;
    g.push_back({5, chars("012aceiost")});
    g.push_back({6, chars(" %-./3456789=A_bdfghlmnpru")});
    g.push_back({7, chars(":BCDEFGHIJKLMNOPQRSTUVWYjkqvwxyz")});
    g.push_back({8, chars("&*,;XZ")});
    g.push_back({10, chars("!\"()?")});
    g.push_back({11, chars("'+|")});
    g.push_back({12, chars("#>")});
    g.push_back({13, {0, '$', '@', '[', ']', '~'}});
    g.push_back({14, chars("^}")});
    g.push_back({15, chars("<`{")});
    g.push_back({19, {'\\', 195, 208}});
    g.push_back({20, {128, 130, 131, 162, 184, 194, 224, 226}});
    g.push_back({21, {153, 161, 167, 172, 176, 177, 179, 209, 216, 217, 227, 229, 230}});
    g.push_back({22, {129, 132, 133, 134, 136, 146, 154, 156, 160, 163, 164, 169, 170, 173, 178, 181, 185,
                      186, 187, 189, 190, 196, 198, 228, 232, 233}});
    g.push_back({23, {1,   135, 137, 138, 139, 140, 141, 143, 147, 149, 150, 151, 152, 155, 157,
                      158, 165, 166, 168, 174, 175, 180, 182, 183, 188, 191, 197, 231, 239}});
    g.push_back({24, {9, 142, 144, 145, 148, 159, 171, 206, 215, 225, 236, 237}});
    g.push_back({25, {199, 207, 234, 235}});
    g.push_back({26, {192, 193, 200, 201, 202, 205, 210, 213, 218, 219, 238, 240, 242, 243, 255}});
    g.push_back({27, {203, 204, 211, 212, 214, 221, 222, 223, 241, 244, 245, 246, 247, 248, 250, 251, 252, 253, 254}});
    g.push_back({28, {2,  3,  4,  5,  6,  7,  8,  11, 12, 14, 15, 16, 17, 18, 19,
                      20, 21, 23, 24, 25, 26, 27, 28, 29, 30, 31, 127, 220, 249}});
    g.push_back({30, {10, 13, 22, 256}});
    for (auto& grp : g) std::sort(grp.symbols.begin(), grp.symbols.end());
    return g;
  }();
  return groups;
}

struct HuffmanTables {
  uint32_t code[257];
  uint8_t bits[257];
  // binary decode tree: child[node][bit]; negative = -(symbol + 1); 0 = absent
  std::vector<std::array<int, 2>> tree;
  bool valid = false;

  HuffmanTables() {
    std::memset(code, 0, sizeof(code));
    std::memset(bits, 0, sizeof(bits));
    uint64_t next = 0;
    int prev_bits = 0;
    int count = 0;
    for (const auto& grp : length_groups()) {
      next <<= (grp.bits - prev_bits);
      prev_bits = grp.bits;
      for (int sym : grp.symbols) {
        code[sym] = static_cast<uint32_t>(next++);
        bits[sym] = static_cast<uint8_t>(grp.bits);
        ++count;
      }
    }
    // a complete prefix code ends exactly at 2^30 after the last 30-bit code
    valid = (count == 257) && (next == (1ull << 30));
    tree.push_back({0, 0});
    for (int sym = 0; sym < 257; ++sym) {
      int node = 0;
      for (int b = bits[sym] - 1; b >= 0; --b) {
        const int bit = (code[sym] >> b) & 1;
        if (b == 0) {
          tree[node][bit] = -(sym + 1);
        } else {
          if (tree[node][bit] == 0) {
            tree.push_back({0, 0});
            tree[node][bit] = static_cast<int>(tree.size()) - 1;
          }
          node = tree[node][bit];
        }
      }
    }
  }
};

const HuffmanTables& huffman() {
  static const HuffmanTables t;
  return t;
}

// ---- integers and strings (RFC 7541 section 5)
void put_int(std::string* out, uint8_t first_byte_flags, int prefix_bits, uint64_t value) {
  const uint64_t max_prefix = (1u << prefix_bits) - 1;
  if (value < max_prefix) {
    out->push_back(static_cast<char>(first_byte_flags | value));
    return;
  }
  out->push_back(static_cast<char>(first_byte_flags | max_prefix));
  value -= max_prefix;
  while (value >= 128) {
    out->push_back(static_cast<char>((value & 0x7f) | 0x80));
    value >>= 7;
  }
  out->push_back(static_cast<char>(value));
}

bool get_int(const std::string& s, size_t* pos, int prefix_bits, uint64_t* value) {
  if (*pos >= s.size()) return false;
  const uint64_t max_prefix = (1u << prefix_bits) - 1;
  uint64_t v = static_cast<uint8_t>(s[(*pos)++]) & max_prefix;
  if (v < max_prefix) {
    *value = v;
    return true;
  }
  int shift = 0;
  while (true) {
    if (*pos >= s.size() || shift > 56) return false;
    const uint8_t b = static_cast<uint8_t>(s[(*pos)++]);
    v += static_cast<uint64_t>(b & 0x7f) << shift;
    shift += 7;
    if (!(b & 0x80)) break;
  }
  *value = v;
  return true;
}

void put_string(std::string* out, const std::string& s, bool use_huffman) {
  if (use_huffman) {
    const std::string enc = huffman_encode(s);
    if (enc.size() < s.size()) {
      put_int(out, 0x80, 7, enc.size());
      out->append(enc);
      return;
    }
  }
  put_int(out, 0x00, 7, s.size());
  out->append(s);
}

bool get_string(const std::string& s, size_t* pos, std::string* out) {
  if (*pos >= s.size()) return false;
  const bool huff = (static_cast<uint8_t>(s[*pos]) & 0x80) != 0;
  uint64_t len = 0;
  if (!get_int(s, pos, 7, &len)) return false;
  if (len > s.size() - *pos) return false;
  if (huff) {
    if (!huffman_decode(reinterpret_cast<const uint8_t*>(s.data()) + *pos, static_cast<size_t>(len), out)) return false;
  } else {
    out->assign(s, *pos, static_cast<size_t>(len));
  }
  *pos += static_cast<size_t>(len);
  return true;
}

const std::vector<Header>& static_table() {
  static const std::vector<Header> t = {
      {":authority", ""}, {":method", "GET"}, {":method", "POST"}, {":path", "/"}, {":path", "/index.html"},
      {":scheme", "http"}, {":scheme", "https"}, {":status", "200"}, {":status", "204"}, {":status", "206"},
      {":status", "304"}, {":status", "400"}, {":status", "404"}, {":status", "500"}, {"accept-charset", ""},
      {"accept-encoding", "gzip, deflate"}, {"accept-language", ""}, {"accept-ranges", ""}, {"accept", ""},
      {"access-control-allow-origin", ""}, {"age", ""}, {"allow", ""}, {"authorization", ""}, {"cache-control", ""},
      {"content-disposition", ""}, {"content-encoding", ""}, {"content-language", ""}, {"content-length", ""},
      {"content-location", ""}, {"content-range", ""}, {"content-type", ""}, {"cookie", ""}, {"date", ""}, {"etag", ""},
      {"expect", ""}, {"expires", ""}, {"from", ""}, {"host", ""}, {"if-match", ""}, {"if-modified-since", ""},
      {"if-none-match", ""}, {"if-range", ""}, {"if-unmodified-since", ""}, {"last-modified", ""}, {"link", ""},
      {"location", ""}, {"max-forwards", ""}, {"proxy-authenticate", ""}, {"proxy-authorization", ""}, {"range", ""},
      {"referer", ""}, {"refresh", ""}, {"retry-after", ""}, {"server", ""}, {"set-cookie", ""},
      {"strict-transport-security", ""}, {"transfer-encoding", ""}, {"user-agent", ""}, {"vary", ""}, {"via", ""},
      {"www-authenticate", ""}};
  return t;
}

}  // namespace

bool huffman_decode(const uint8_t* data, size_t n, std::string* out) {
  const HuffmanTables& t = huffman();
  out->clear();
  int node = 0;
  int pending_bits = 0;     // bits consumed since the last symbol
  bool pending_all_ones = true;
  for (size_t i = 0; i < n; ++i) {
    for (int b = 7; b >= 0; --b) {
      const int bit = (data[i] >> b) & 1;
      const int next = t.tree[node][bit];
      if (next == 0) return false;
      ++pending_bits;
      pending_all_ones = pending_all_ones && bit;
      if (next < 0) {
        const int sym = -next - 1;
        if (sym == 256) return false;  // an explicit end-of-string symbol is an error
        out->push_back(static_cast<char>(sym));
        node = 0;
        pending_bits = 0;
        pending_all_ones = true;
      } else {
        node = next;
      }
    }
  }
  // padding: fewer than 8 bits, all ones
  return pending_bits < 8 && pending_all_ones;
}

std::string huffman_encode(const std::string& s) {
  const HuffmanTables& t = huffman();
  std::string out;
  uint64_t acc = 0;
  int nbits = 0;
  for (unsigned char c : s) {
    acc = (acc << t.bits[c]) | t.code[c];
    nbits += t.bits[c];
    while (nbits >= 8) {
      out.push_back(static_cast<char>((acc >> (nbits - 8)) & 0xff));
      nbits -= 8;
    }
    acc &= (1ull << nbits) - 1;
  }
  if (nbits > 0) out.push_back(static_cast<char>(((acc << (8 - nbits)) | ((1u << (8 - nbits)) - 1)) & 0xff));
  return out;
}

// ================================================================ HPACK: header blocks
bool HpackDecoder::lookup(uint64_t index, Header* h) const {
  const auto& st = static_table();
  if (index == 0) return false;
  if (index <= st.size()) {
    *h = st[index - 1];
    return true;
  }
  const uint64_t d = index - st.size() - 1;
  if (d >= dynamic_.size()) return false;
  *h = dynamic_[d];
  return true;
}

void HpackDecoder::evict() {
  while (dynamic_bytes_ > max_bytes_ && !dynamic_.empty()) {
    dynamic_bytes_ -= dynamic_.back().name.size() + dynamic_.back().value.size() + 32;
    dynamic_.pop_back();
  }
}

void HpackDecoder::insert(const Header& h) {
  const size_t sz = h.name.size() + h.value.size() + 32;
  if (sz > max_bytes_) {  // larger than the table: empties it
    dynamic_.clear();
    dynamic_bytes_ = 0;
    return;
  }
  dynamic_.push_front(h);
  dynamic_bytes_ += sz;
  evict();
}

bool HpackDecoder::decode(const std::string& block, std::vector<Header>* out) {
  size_t pos = 0;
  while (pos < block.size()) {
    const uint8_t b = static_cast<uint8_t>(block[pos]);
    if (b & 0x80) {  // indexed field
      uint64_t idx;
      Header h;
      if (!get_int(block, &pos, 7, &idx) || !lookup(idx, &h)) return false;
      out->push_back(h);
    } else if ((b & 0xe0) == 0x20) {  // dynamic table size update
      uint64_t sz;
      if (!get_int(block, &pos, 5, &sz) || sz > protocol_max_) return false;
      max_bytes_ = static_cast<size_t>(sz);
      evict();
    } else {
      const bool indexing = (b & 0xc0) == 0x40;
      const int prefix = indexing ? 6 : 4;
      uint64_t idx;
      Header h;
      if (!get_int(block, &pos, prefix, &idx)) return false;
      if (idx != 0) {
        Header named;
        if (!lookup(idx, &named)) return false;
        h.name = named.name;
      } else if (!get_string(block, &pos, &h.name)) {
        return false;
      }
      if (!get_string(block, &pos, &h.value)) return false;
      if (indexing) insert(h);
      out->push_back(h);
    }
  }
  return true;
}

std::string hpack_encode(const std::vector<Header>& headers, bool use_huffman) {
  std::string out;
  const auto& st = static_table();
  for (const Header& h : headers) {
    // exact static matches become one byte; known names are referenced by index
    size_t name_idx = 0;
    bool exact = false;
    for (size_t i = 0; i < st.size(); ++i) {
      if (st[i].name != h.name) continue;
      if (name_idx == 0) name_idx = i + 1;
      if (!st[i].value.empty() && st[i].value == h.value) {
        put_int(&out, 0x80, 7, i + 1);
        exact = true;
        break;
      }
    }
    if (exact) continue;
    put_int(&out, 0x00, 4, name_idx);  // literal without indexing
    if (name_idx == 0) put_string(&out, h.name, use_huffman);
    put_string(&out, h.value, use_huffman);
  }
  return out;
}

std::string percent_encode(const std::string& s) {
  static const char* hex = "0123456789ABCDEF";
  std::string out;
  for (unsigned char c : s) {
    if (c >= 0x20 && c <= 0x7e && c != '%') {
      out.push_back(static_cast<char>(c));
    } else {
      out.push_back('%');
      out.push_back(hex[c >> 4]);
      out.push_back(hex[c & 15]);
    }
  }
  return out;
}

std::string percent_decode(const std::string& s) {
  auto hexval = [](char c) -> int {
    if (c >= '0' && c <= '9') return c - '0';
    if (c >= 'a' && c <= 'f') return c - 'a' + 10;
    if (c >= 'A' && c <= 'F') return c - 'A' + 10;
    return -1;
  };
  std::string out;
  for (size_t i = 0; i < s.size(); ++i) {
    if (s[i] == '%' && i + 2 < s.size() && hexval(s[i + 1]) >= 0 && hexval(s[i + 2]) >= 0) {
      out.push_back(static_cast<char>(hexval(s[i + 1]) * 16 + hexval(s[i + 2])));
      i += 2;
    } else {
      out.push_back(s[i]);
    }
  }
  return out;
}

// ================================================================ HTTP/2 framing
namespace {

enum FrameType : uint8_t {
  kData = 0, kHeaders = 1, kPriority = 2, kRstStream = 3, kSettings = 4, kPushPromise = 5, kPing = 6, kGoAway = 7,
  kWindowUpdate = 8, kContinuation = 9,
};
constexpr uint8_t kFlagEndStream = 0x1, kFlagAck = 0x1, kFlagEndHeaders = 0x4, kFlagPadded = 0x8, kFlagPriority = 0x20;
constexpr uint16_t kSettingsHeaderTableSize = 1, kSettingsInitialWindowSize = 4, kSettingsMaxFrameSize = 5;
constexpr uint32_t kErrProtocol = 1, kErrRefusedStream = 7, kErrCancel = 8, kErrCompression = 9;
constexpr size_t kMaxOpenStreams = 1024;  // calls in progress per connection (advertised in SETTINGS)
constexpr uint16_t kSettingsMaxConcurrentStreams = 3;
const char kPreface[] = "PRI * HTTP/2.0\r\n\r\nSM\r\n\r\n";
constexpr size_t kPrefaceLen = 24;
constexpr uint32_t kMaxMessageBytes = 64u << 20;

struct Frame {
  uint8_t type = 0, flags = 0;
  uint32_t stream = 0;
  std::string payload;
};

std::string frame_bytes(uint8_t type, uint8_t flags, uint32_t stream, const std::string& payload) {
  std::string out;
  const uint32_t n = static_cast<uint32_t>(payload.size());
  out.push_back(static_cast<char>((n >> 16) & 0xff));
  out.push_back(static_cast<char>((n >> 8) & 0xff));
  out.push_back(static_cast<char>(n & 0xff));
  out.push_back(static_cast<char>(type));
  out.push_back(static_cast<char>(flags));
  out.push_back(static_cast<char>((stream >> 24) & 0x7f));
  out.push_back(static_cast<char>((stream >> 16) & 0xff));
  out.push_back(static_cast<char>((stream >> 8) & 0xff));
  out.push_back(static_cast<char>(stream & 0xff));
  out.append(payload);
  return out;
}

std::string u32_bytes(uint32_t v) {
  std::string s;
  s.push_back(static_cast<char>((v >> 24) & 0xff));
  s.push_back(static_cast<char>((v >> 16) & 0xff));
  s.push_back(static_cast<char>((v >> 8) & 0xff));
  s.push_back(static_cast<char>(v & 0xff));
  return s;
}

uint32_t read_u32(const std::string& s, size_t off) {
  return (static_cast<uint32_t>(static_cast<uint8_t>(s[off])) << 24) | (static_cast<uint32_t>(static_cast<uint8_t>(s[off + 1])) << 16) |
         (static_cast<uint32_t>(static_cast<uint8_t>(s[off + 2])) << 8) | static_cast<uint32_t>(static_cast<uint8_t>(s[off + 3]));
}

// Reads one frame; kIoTimeout only when a deadline is given.
IoResult read_frame(int fd, Frame* f, Clock::time_point deadline, const std::atomic<bool>* stopping) {
  char hdr[9];
  IoResult r = read_exact(fd, hdr, 9, deadline, stopping);
  if (r != kIoOk) return r;
  const uint8_t* u = reinterpret_cast<const uint8_t*>(hdr);
  const uint32_t len = (static_cast<uint32_t>(u[0]) << 16) | (static_cast<uint32_t>(u[1]) << 8) | u[2];
  f->type = u[3];
  f->flags = u[4];
  f->stream = ((static_cast<uint32_t>(u[5]) & 0x7f) << 24) | (static_cast<uint32_t>(u[6]) << 16) |
              (static_cast<uint32_t>(u[7]) << 8) | u[8];
  if (len > (1u << 24)) return kIoClosed;
  f->payload.assign(len, '\0');
  if (len == 0) return kIoOk;
  const Clock::time_point body_deadline =
      deadline == Clock::time_point::max() ? Clock::now() + std::chrono::seconds(30) : deadline;
  return read_exact(fd, &f->payload[0], len, body_deadline, stopping);
}

// Strips padding and the priority block of a HEADERS frame; false on a malformed frame.
bool headers_fragment(const Frame& f, std::string* fragment) {
  size_t off = 0, end = f.payload.size();
  if (f.flags & kFlagPadded) {
    if (end < 1) return false;
    const size_t pad = static_cast<uint8_t>(f.payload[0]);
    off = 1;
    if (pad > end - off) return false;
    end -= pad;
  }
  if (f.flags & kFlagPriority) {
    if (end - off < 5) return false;
    off += 5;
  }
  fragment->assign(f.payload, off, end - off);
  return true;
}

bool data_payload(const Frame& f, std::string* data) {
  size_t off = 0, end = f.payload.size();
  if (f.flags & kFlagPadded) {
    if (end < 1) return false;
    const size_t pad = static_cast<uint8_t>(f.payload[0]);
    off = 1;
    if (pad > end - off) return false;
    end -= pad;
  }
  data->append(f.payload, off, end - off);
  return true;
}

std::string grpc_frame(const std::string& message) {
  std::string out;
  out.push_back('\0');  // not compressed
  out.append(u32_bytes(static_cast<uint32_t>(message.size())));
  out.append(message);
  return out;
}

// Extracts the single message of a unary call; false if the framing is wrong or compressed.
bool grpc_unframe(const std::string& data, std::string* message) {
  if (data.size() < 5 || data[0] != '\0') return false;
  const uint32_t len = read_u32(data, 1);
  if (len != data.size() - 5) return false;
  message->assign(data, 5, len);
  return true;
}

const std::string* find_header(const std::vector<Header>& hs, const std::string& name) {
  for (const Header& h : hs)
    if (h.name == name) return &h.value;
  return nullptr;
}

// ---------------------------------------------------------------- server connection
struct ServerStream {
  std::vector<Header> headers;
  std::string data;
  bool headers_done = false;
  int64_t send_window = 65535;
  std::shared_ptr<std::atomic<bool>> cancelled = std::make_shared<std::atomic<bool>>(false);
};

struct ServerConn {
  int fd;
  const std::atomic<bool>* stopping;
  std::mutex mu;  // guards writes, windows and the stream table
  std::condition_variable window_cv;
  int64_t conn_send_window = 65535;
  int64_t peer_initial_window = 65535;
  uint32_t peer_max_frame = 16384;
  std::map<uint32_t, ServerStream> streams;
  std::atomic<bool> dead{false};
  int handlers = 0;
  std::condition_variable handlers_cv;

  bool send_locked(const std::string& bytes) {
    if (dead.load()) return false;
    if (write_all(fd, bytes.data(), bytes.size(), Clock::now() + std::chrono::seconds(30)) != kIoOk) {
      dead.store(true);
      return false;
    }
    return true;
  }
  bool send(const std::string& bytes) {
    std::lock_guard<std::mutex> g(mu);
    return send_locked(bytes);
  }
};

// Sends response headers, the message (respecting flow control) and the trailers of one call.
void respond(ServerConn* c, uint32_t stream, const Status& st, const std::string& message) {
  std::unique_lock<std::mutex> lk(c->mu);
  auto it = c->streams.find(stream);
  if (it == c->streams.end() || it->second.cancelled->load()) {
    c->streams.erase(stream);
    return;
  }
  std::vector<Header> trailers = {{"grpc-status", std::to_string(st.code)}};
  if (!st.message.empty()) trailers.push_back({"grpc-message", percent_encode(st.message)});
  if (!st.ok()) {
    // trailers-only response
    std::vector<Header> hs = {{":status", "200"}, {"content-type", "application/grpc"}};
    hs.insert(hs.end(), trailers.begin(), trailers.end());
    c->send_locked(frame_bytes(kHeaders, kFlagEndHeaders | kFlagEndStream, stream, hpack_encode(hs, false)));
    c->streams.erase(stream);
    return;
  }
  const std::string head = frame_bytes(kHeaders, kFlagEndHeaders, stream,
                                       hpack_encode({{":status", "200"}, {"content-type", "application/grpc"}}, false));
  const std::string body = grpc_frame(message);
  // common case: the whole message fits one frame and both windows, so headers, message and trailers
  // leave in a single write
  if (body.size() <= c->peer_max_frame && static_cast<int64_t>(body.size()) <= c->conn_send_window &&
      static_cast<int64_t>(body.size()) <= it->second.send_window) {
    c->conn_send_window -= static_cast<int64_t>(body.size());
    c->send_locked(head + frame_bytes(kData, 0, stream, body) +
                   frame_bytes(kHeaders, kFlagEndHeaders | kFlagEndStream, stream, hpack_encode(trailers, false)));
    c->streams.erase(stream);
    return;
  }
  c->send_locked(head);
  size_t off = 0;
  const Clock::time_point give_up = Clock::now() + std::chrono::seconds(60);
  while (off < body.size() && !c->dead.load()) {
    it = c->streams.find(stream);
    if (it == c->streams.end() || it->second.cancelled->load()) break;
    const int64_t window = std::min(c->conn_send_window, it->second.send_window);
    if (window <= 0) {
      if (c->window_cv.wait_until(lk, give_up) == std::cv_status::timeout) break;
      continue;
    }
    const size_t n = std::min<size_t>({body.size() - off, static_cast<size_t>(window), c->peer_max_frame});
    c->conn_send_window -= static_cast<int64_t>(n);
    it->second.send_window -= static_cast<int64_t>(n);
    if (!c->send_locked(frame_bytes(kData, 0, stream, body.substr(off, n)))) break;
    off += n;
  }
  if (off == body.size())
    c->send_locked(frame_bytes(kHeaders, kFlagEndHeaders | kFlagEndStream, stream, hpack_encode(trailers, false)));
  else if (!c->dead.load())
    c->send_locked(frame_bytes(kRstStream, 0, stream, u32_bytes(kErrCancel)));
  c->streams.erase(stream);
}

}  // namespace

void serve_connection(int fd, const std::string& prefix, const std::atomic<bool>& stopping, const Dispatch& dispatch) {
  // the rest of the client preface
  if (prefix.size() > kPrefaceLen || std::memcmp(prefix.data(), kPreface, prefix.size()) != 0) return;
  std::string rest(kPrefaceLen - prefix.size(), '\0');
  if (!rest.empty() &&
      read_exact(fd, &rest[0], rest.size(), Clock::now() + std::chrono::seconds(10), &stopping) != kIoOk)
    return;
  if (std::memcmp(rest.data(), kPreface + prefix.size(), rest.size()) != 0) return;

  auto conn = std::make_shared<ServerConn>();
  conn->fd = fd;
  conn->stopping = &stopping;
  {
    std::string settings;
    settings.push_back(static_cast<char>(kSettingsMaxConcurrentStreams >> 8));
    settings.push_back(static_cast<char>(kSettingsMaxConcurrentStreams & 0xff));
    settings.append(u32_bytes(static_cast<uint32_t>(kMaxOpenStreams)));
    if (!conn->send(frame_bytes(kSettings, 0, 0, settings))) return;
  }

  HpackDecoder decoder;
  uint32_t continuation_stream = 0;  // non-zero while a header block is open
  std::string header_block;
  bool block_ends_stream = false;
  uint32_t last_stream = 0;

  auto finish = [&] {
    conn->dead.store(true);
    std::unique_lock<std::mutex> lk(conn->mu);
    for (auto& kv : conn->streams) kv.second.cancelled->store(true);
    conn->window_cv.notify_all();
    conn->handlers_cv.wait_for(lk, std::chrono::seconds(10), [&] { return conn->handlers == 0; });
  };
  auto goaway = [&](uint32_t code) {
    conn->send(frame_bytes(kGoAway, 0, 0, u32_bytes(last_stream) + u32_bytes(code)));
  };
  // Runs the handler of a complete request in its own thread: quorum calls block for a long time.
  auto start_call = [&](uint32_t id) {
    std::vector<Header> headers;
    std::string data;
    std::shared_ptr<std::atomic<bool>> cancelled;
    {
      std::lock_guard<std::mutex> g(conn->mu);
      ServerStream& s = conn->streams[id];
      headers = s.headers;
      data.swap(s.data);
      cancelled = s.cancelled;
      ++conn->handlers;
    }
    std::thread([conn, id, headers, data, cancelled, dispatch, &stopping] {
      Status st;
      std::string resp, message;
      const std::string* path = find_header(headers, ":path");
      const std::string* tmo = find_header(headers, "grpc-timeout");
      const std::string* ctype = find_header(headers, "content-type");
      CallContext ctx;
      ctx.stopping = &stopping;
      ctx.stream_cancelled = cancelled.get();
      if (tmo != nullptr) {
        ctx.timeout = parse_grpc_timeout(*tmo);
        if (ctx.timeout) ctx.deadline = Clock::now() + std::chrono::duration_cast<Clock::duration>(*ctx.timeout);
      }
      if (path == nullptr || ctype == nullptr || ctype->compare(0, 16, "application/grpc") != 0) {
        st = Status::Error(kInvalidArgument, "not a gRPC request");
      } else if (tmo != nullptr && !ctx.timeout) {
        st = Status::Error(kInvalidArgument, "invalid timeout " + *tmo);
      } else if (!data.empty() && data[0] == '\1') {
        st = Status::Error(12 /*Unimplemented*/, "message compression is not supported (send grpc-encoding: identity)");
      } else if (!grpc_unframe(data, &message)) {
        st = Status::Error(kInternal, "malformed gRPC message");
      } else {
        try {
          st = dispatch(*path, ctx, message, &resp);
        } catch (const std::exception& e) {
          st = Status::Error(kInternal, e.what());
        }
      }
      respond(conn.get(), id, st, resp);
      std::lock_guard<std::mutex> g(conn->mu);
      --conn->handlers;
      conn->handlers_cv.notify_all();
    }).detach();
  };

  while (!stopping.load() && !conn->dead.load()) {
    Frame f;
    if (read_frame(fd, &f, Clock::time_point::max(), &stopping) != kIoOk) break;
    if (continuation_stream != 0 && (f.type != kContinuation || f.stream != continuation_stream)) {
      goaway(kErrProtocol);
      break;
    }
    bool block_complete = false;
    switch (f.type) {
      case kSettings: {
        if (f.flags & kFlagAck) break;
        if (f.payload.size() % 6 != 0) { goaway(kErrProtocol); conn->dead.store(true); break; }
        std::lock_guard<std::mutex> g(conn->mu);
        for (size_t i = 0; i + 6 <= f.payload.size(); i += 6) {
          const uint16_t id = static_cast<uint16_t>((static_cast<uint8_t>(f.payload[i]) << 8) | static_cast<uint8_t>(f.payload[i + 1]));
          const uint32_t v = read_u32(f.payload, i + 2);
          if (id == kSettingsInitialWindowSize) {
            const int64_t delta = static_cast<int64_t>(v) - conn->peer_initial_window;
            conn->peer_initial_window = v;
            for (auto& kv : conn->streams) kv.second.send_window += delta;
          } else if (id == kSettingsMaxFrameSize && v >= 16384 && v <= 16777215) {
            conn->peer_max_frame = v;
          }
        }
        conn->send_locked(frame_bytes(kSettings, kFlagAck, 0, ""));
        conn->window_cv.notify_all();
        break;
      }
      case kPing:
        if (!(f.flags & kFlagAck) && f.payload.size() == 8) conn->send(frame_bytes(kPing, kFlagAck, 0, f.payload));
        break;
      case kWindowUpdate: {
        if (f.payload.size() != 4) break;
        const uint32_t inc = read_u32(f.payload, 0) & 0x7fffffffu;
        std::lock_guard<std::mutex> g(conn->mu);
        if (f.stream == 0) {
          conn->conn_send_window += inc;
        } else {
          auto it = conn->streams.find(f.stream);
          if (it != conn->streams.end()) it->second.send_window += inc;
        }
        conn->window_cv.notify_all();
        break;
      }
      case kRstStream: {
        std::lock_guard<std::mutex> g(conn->mu);
        auto it = conn->streams.find(f.stream);
        if (it != conn->streams.end()) it->second.cancelled->store(true);
        conn->window_cv.notify_all();
        break;
      }
      case kGoAway:
        conn->dead.store(true);
        break;
      case kHeaders: {
        if (f.stream == 0 || (f.stream & 1) == 0) { goaway(kErrProtocol); conn->dead.store(true); break; }
        header_block.clear();
        if (!headers_fragment(f, &header_block)) { goaway(kErrProtocol); conn->dead.store(true); break; }
        block_ends_stream = (f.flags & kFlagEndStream) != 0;
        last_stream = std::max(last_stream, f.stream);
        {
          std::lock_guard<std::mutex> g(conn->mu);
          ServerStream& s = conn->streams[f.stream];
          if (!s.headers_done) s.send_window = conn->peer_initial_window;
        }
        if (f.flags & kFlagEndHeaders) block_complete = true; else continuation_stream = f.stream;
        break;
      }
      case kContinuation:
        if (continuation_stream == 0) { goaway(kErrProtocol); conn->dead.store(true); break; }
        header_block.append(f.payload);
        if (f.flags & kFlagEndHeaders) { block_complete = true; continuation_stream = 0; }
        break;
      case kData: {
        std::string chunk;
        if (!data_payload(f, &chunk)) { goaway(kErrProtocol); conn->dead.store(true); break; }
        bool known = false, too_big = false;
        {
          std::lock_guard<std::mutex> g(conn->mu);
          auto it = conn->streams.find(f.stream);
          if (it != conn->streams.end() && it->second.headers_done) {
            known = true;
            it->second.data.append(chunk);
            too_big = it->second.data.size() > kMaxMessageBytes;
          }
          // give the consumed bytes back to the sender's windows
          if (!f.payload.empty()) {
            const std::string inc = u32_bytes(static_cast<uint32_t>(f.payload.size()));
            conn->send_locked(frame_bytes(kWindowUpdate, 0, 0, inc));
            if (known && !(f.flags & kFlagEndStream)) conn->send_locked(frame_bytes(kWindowUpdate, 0, f.stream, inc));
          }
        }
        if (too_big) { goaway(kErrProtocol); conn->dead.store(true); break; }
        if (known && (f.flags & kFlagEndStream)) start_call(f.stream);
        break;
      }
      default:
        break;  // PRIORITY, PUSH_PROMISE (never valid from a client) and unknown types are ignored
    }
    if (block_complete) {
      const uint32_t id = f.stream;
      std::vector<Header> decoded;
      if (!decoder.decode(header_block, &decoded)) {
        goaway(kErrCompression);
        break;
      }
      bool ready = false;
      {
        std::lock_guard<std::mutex> g(conn->mu);
        if (conn->streams.size() > kMaxOpenStreams) {
          // the block had to be decoded (the compression state is per connection); the call is refused
          conn->streams.erase(id);
          conn->send_locked(frame_bytes(kRstStream, 0, id, u32_bytes(kErrRefusedStream)));
          continue;
        }
        ServerStream& s = conn->streams[id];
        if (!s.headers_done) {
          s.headers = decoded;
          s.headers_done = true;
        }  // a second block would be request trailers: nothing in them matters here
        ready = block_ends_stream;
      }
      if (ready) start_call(id);
    }
  }
  finish();
}

// ================================================================ client
ClientConnection::ClientConnection(int fd, const std::string& authority) : fd_(fd), authority_(authority) {}

ClientConnection::~ClientConnection() {
  if (fd_ >= 0) {
    if (ready_) {
      const std::string bye = frame_bytes(kGoAway, 0, 0, u32_bytes(0) + u32_bytes(0));
      write_all(fd_, bye.data(), bye.size(), Clock::now() + std::chrono::milliseconds(200));
    }
    ::close(fd_);
  }
}

bool ClientConnection::handshake() {
  if (ready_) return true;
  std::string hello(kPreface, kPrefaceLen);
  hello += frame_bytes(kSettings, 0, 0, "");
  if (write_all(fd_, hello.data(), hello.size(), Clock::now() + std::chrono::seconds(10)) != kIoOk) return false;
  ready_ = true;  // the server's SETTINGS frame is handled by the read loop of the first call
  return true;
}

Status ClientConnection::call(const std::string& path, const std::string& payload, std::optional<Millis> timeout,
                              std::string* resp, bool* broken) {
  *broken = false;
  auto fail = [&](int code, const std::string& msg) {
    *broken = true;
    return Status::Error(code, msg);
  };
  if (!handshake()) return fail(kUnavailable, "connection closed during the HTTP/2 preface");
  const Clock::time_point deadline = timeout ? Clock::now() + *timeout : Clock::time_point::max();
  const uint32_t id = next_stream_;
  next_stream_ += 2;
  if (next_stream_ > 0x7ffffff0u) *broken = true;  // stream ids are used up: the caller reconnects next time

  std::vector<Header> hs = {{":method", "POST"}, {":scheme", "http"}, {":path", path}, {":authority", authority_},
                            {"te", "trailers"}, {"content-type", "application/grpc"},
                            {"user-agent", "torchft_b200-control/1"}};
  if (timeout) hs.push_back({"grpc-timeout", format_grpc_timeout(*timeout)});
  std::string out = frame_bytes(kHeaders, kFlagEndHeaders, id, hpack_encode(hs, true));
  // Requests of this control plane are a few hundred bytes; larger ones are cut to the peer's frame size
  // and must fit the initial windows (65535 bytes) because the call is written before anything is read.
  const std::string body = grpc_frame(payload);
  if (static_cast<int64_t>(body.size()) > std::min(conn_send_window_, peer_initial_window_))
    return Status::Error(kInvalidArgument, "request larger than the HTTP/2 flow-control window");
  conn_send_window_ -= static_cast<int64_t>(body.size());
  size_t off = 0;
  do {
    const size_t n = std::min<size_t>(body.size() - off, peer_max_frame_);
    const bool last = off + n == body.size();
    out += frame_bytes(kData, last ? kFlagEndStream : 0, id, body.substr(off, n));
    off += n;
  } while (off < body.size());
  if (write_all(fd_, out.data(), out.size(), deadline) != kIoOk) return fail(kUnavailable, "connection lost while sending");

  std::vector<Header> response_headers, trailers;
  std::string data, block;
  uint32_t open_block = 0;
  bool block_end_stream = false;
  bool stream_closed = false;
  while (!stream_closed) {
    Frame f;
    const IoResult r = read_frame(fd_, &f, deadline, nullptr);
    if (r == kIoTimeout) {
      const std::string rst = frame_bytes(kRstStream, 0, id, u32_bytes(kErrCancel));
      if (write_all(fd_, rst.data(), rst.size(), Clock::now() + std::chrono::seconds(1)) != kIoOk) *broken = true;
      return Status::Error(kCancelled, "Timeout expired");
    }
    if (r != kIoOk) return fail(kUnavailable, "connection closed by the server");
    bool block_complete = false;
    switch (f.type) {
      case kSettings: {
        if (f.flags & kFlagAck) break;
        for (size_t i = 0; i + 6 <= f.payload.size(); i += 6) {
          const uint16_t sid = static_cast<uint16_t>((static_cast<uint8_t>(f.payload[i]) << 8) | static_cast<uint8_t>(f.payload[i + 1]));
          const uint32_t v = read_u32(f.payload, i + 2);
          if (sid == kSettingsInitialWindowSize) peer_initial_window_ = v;
          if (sid == kSettingsMaxFrameSize && v >= 16384 && v <= 16777215) peer_max_frame_ = v;
        }
        const std::string ack = frame_bytes(kSettings, kFlagAck, 0, "");
        if (write_all(fd_, ack.data(), ack.size(), Clock::now() + std::chrono::seconds(5)) != kIoOk)
          return fail(kUnavailable, "connection lost");
        break;
      }
      case kPing:
        if (!(f.flags & kFlagAck) && f.payload.size() == 8) {
          const std::string pong = frame_bytes(kPing, kFlagAck, 0, f.payload);
          if (write_all(fd_, pong.data(), pong.size(), Clock::now() + std::chrono::seconds(5)) != kIoOk)
            return fail(kUnavailable, "connection lost");
        }
        break;
      case kWindowUpdate:
        if (f.payload.size() == 4 && f.stream == 0) conn_send_window_ += read_u32(f.payload, 0) & 0x7fffffffu;
        break;
      case kGoAway:
        // calls above the server's last stream id were not processed; ours may still complete
        if (f.payload.size() >= 4 && (read_u32(f.payload, 0) & 0x7fffffffu) < id)
          return fail(kUnavailable, "server is going away");
        *broken = true;
        break;
      case kRstStream:
        if (f.stream == id) return Status::Error(kUnavailable, "stream reset by the server");
        break;
      case kHeaders:
        block.clear();
        if (!headers_fragment(f, &block)) return fail(kInternal, "malformed HEADERS frame");
        open_block = f.stream;
        block_end_stream = (f.flags & kFlagEndStream) != 0;
        if (f.flags & kFlagEndHeaders) block_complete = true;
        break;
      case kContinuation:
        if (f.stream != open_block) return fail(kInternal, "unexpected CONTINUATION frame");
        block.append(f.payload);
        if (f.flags & kFlagEndHeaders) block_complete = true;
        break;
      case kData: {
        if (f.stream == id) {
          if (!data_payload(f, &data)) return fail(kInternal, "malformed DATA frame");
          if (data.size() > kMaxMessageBytes) return fail(kInternal, "response too large");
          if (f.flags & kFlagEndStream) stream_closed = true;
        }
        if (!f.payload.empty()) {
          const std::string inc = u32_bytes(static_cast<uint32_t>(f.payload.size()));
          std::string wu = frame_bytes(kWindowUpdate, 0, 0, inc);
          if (f.stream == id && !stream_closed) wu += frame_bytes(kWindowUpdate, 0, id, inc);
          if (write_all(fd_, wu.data(), wu.size(), Clock::now() + std::chrono::seconds(5)) != kIoOk)
            return fail(kUnavailable, "connection lost");
        }
        break;
      }
      default:
        break;
    }
    if (block_complete) {
      // every header block goes through the decoder, whichever stream it belongs to: the table is shared
      std::vector<Header> decoded;
      if (!decoder_.decode(block, &decoded)) return fail(kInternal, "HPACK decoding failed");
      if (open_block == id) {
        if (response_headers.empty() && !block_end_stream) {
          response_headers = decoded;
        } else {
          trailers = decoded;
          if (response_headers.empty()) response_headers = decoded;  // trailers-only response
        }
        if (block_end_stream) stream_closed = true;
      }
      open_block = 0;
    }
  }

  const std::string* http_status = find_header(response_headers, ":status");
  if (http_status == nullptr || *http_status != "200")
    return Status::Error(kUnknown, "unexpected HTTP status " + (http_status ? *http_status : std::string("(none)")));
  const std::string* grpc_status = find_header(trailers, "grpc-status");
  if (grpc_status == nullptr) return Status::Error(kUnknown, "response without grpc-status");
  const int code = std::atoi(grpc_status->c_str());
  if (code != kOk) {
    const std::string* msg = find_header(trailers, "grpc-message");
    return Status::Error(code, msg ? percent_decode(*msg) : std::string());
  }
  if (!grpc_unframe(data, resp)) return Status::Error(kInternal, "malformed or compressed gRPC response");
  return Status::Ok();
}

}  // namespace h2
}  // namespace net
}  // namespace tft

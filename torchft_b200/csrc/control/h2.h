// gRPC over HTTP/2 (cleartext, prior knowledge) for the control plane: the wire format of the
// reference's tonic services (proto/torchft.proto, src/lighthouse.rs:322-360, src/net.rs:8-34),
// so its Rust clients and servers and any stock gRPC stack interoperate with this one.
//
// Contents: HPACK (RFC 7541: static table, dynamic table, integer and string coding, Huffman),
// HTTP/2 framing (RFC 9113: SETTINGS, HEADERS/CONTINUATION, DATA, WINDOW_UPDATE, PING,
// RST_STREAM, GOAWAY) with flow control in both directions, a multiplexing server side that
// runs every request in its own thread, and a unary client.
#pragma once

#include <atomic>
#include <cstdint>
#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <optional>
#include <string>
#include <vector>

#include "net.h"

namespace tft {
namespace net {
namespace h2 {

struct Header {
  std::string name, value;
};

// ---- HPACK
bool huffman_decode(const uint8_t* data, size_t n, std::string* out);  // false on a malformed string
std::string huffman_encode(const std::string& s);

class HpackDecoder {
 public:
  // Decodes one complete header block; false means a compression error (connection must close).
  bool decode(const std::string& block, std::vector<Header>* out);
  void set_max_table_size(size_t n) { protocol_max_ = n; }

 private:
  bool lookup(uint64_t index, Header* h) const;
  void insert(const Header& h);
  void evict();
  std::deque<Header> dynamic_;  // newest first
  size_t dynamic_bytes_ = 0;
  size_t max_bytes_ = 4096;       // current limit (changed by size updates in the block)
  size_t protocol_max_ = 4096;    // SETTINGS_HEADER_TABLE_SIZE we advertised
};

// Encodes headers as literals without indexing (optionally Huffman-coded values); never touches
// a dynamic table, so it is stateless.
std::string hpack_encode(const std::vector<Header>& headers, bool huffman);

// ---- server side: serves one accepted connection until it closes.  `prefix` holds bytes of the
// client preface that the caller already consumed while sniffing the protocol.
using Dispatch =
    std::function<Status(const std::string& path, const CallContext& ctx, const std::string& payload, std::string* resp)>;
void serve_connection(int fd, const std::string& prefix, const std::atomic<bool>& stopping, const Dispatch& dispatch);

// ---- client side: one connection, one call at a time.
class ClientConnection {
 public:
  ClientConnection(int fd, const std::string& authority);
  ~ClientConnection();
  // Returns the status of the call; the response message lands in *resp.  `*broken` is set when the
  // connection cannot be used again.
  Status call(const std::string& path, const std::string& payload, std::optional<Millis> timeout, std::string* resp,
              bool* broken);

 private:
  bool handshake();
  int fd_;
  std::string authority_;
  bool ready_ = false;
  uint32_t next_stream_ = 1;
  uint32_t peer_max_frame_ = 16384;
  int64_t conn_send_window_ = 65535;
  int64_t peer_initial_window_ = 65535;
  HpackDecoder decoder_;
};

std::string percent_encode(const std::string& s);
std::string percent_decode(const std::string& s);

}  // namespace h2
}  // namespace net
}  // namespace tft

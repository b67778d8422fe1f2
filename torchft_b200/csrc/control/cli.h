// Command-line parsing for the lighthouse (flags follow the reference's
// src/lighthouse.rs:66-103: --bind, --join_timeout_ms, --min_replicas,
// --quorum_tick_ms, --heartbeat_timeout_ms).
#pragma once

#include <string>
#include <vector>

#include "quorum.h"

namespace tft {

// Throws std::invalid_argument with a usage message on bad input.
LighthouseOptions parse_lighthouse_args(const std::vector<std::string>& args);
// Blocks forever serving a lighthouse.
int run_lighthouse(const LighthouseOptions& opt);

}  // namespace tft

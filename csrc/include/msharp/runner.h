// The benchmark program as a library: one call per rank process, one call for the launcher.
// The sequence of steps is the reference project's Run() (src/main.cc:389-486) and
// RunAllReduceIteration() (src/main.cc:78-150); what differs is noted in runner.cc.
#pragma once

#include <iosfwd>
#include <string>
#include <vector>

#include "msharp/bootstrap.h"
#include "msharp/config.h"
#include "msharp/driver_api.h"

namespace msharp {

// Runs as rank `comm.rank()`. Rank 0 writes the report to `out`. Returns 0, or 2 when the
// result check failed (agreed by all ranks). Throws on errors.
int run_rank(const Config& cfg, Bootstrap& comm, const DriverApi& api, std::ostream& out);

// Host-only oracle run (no GPU): `rank_count` synthetic ranks of cfg.bytes each are generated,
// reduced on the CPU with both models, and summarised as one JSON line (or text) on `out`.
int run_cpu_only(const Config& cfg, std::ostream& out);

// Fork one child per rank of the plan, running `argv` with RANK / WORLD_SIZE / LOCAL_RANK /
// MSHARP_SESSION set. Returns the first non-zero child status (the other children are then
// terminated by pid), else 0.
int spawn_local_ranks(const std::vector<std::string>& argv, int world, const std::string& session);

// The same for the part of a multi-host job that runs on this host: one child per entry of
// `global_ranks` (RANK = that entry, LOCAL_RANK = its index in the list), WORLD_SIZE = world,
// and MSHARP_HUB_ADDR = hub_address so that every rank reaches rank 0 over TCP.
int spawn_host_ranks(const std::vector<std::string>& argv, int world, const std::string& session,
                     const std::vector<int>& global_ranks, const std::string& hub_address);

}  // namespace msharp

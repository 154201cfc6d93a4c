// mnnvl_sharp_allreduce: the benchmark binary.
//
// Started without RANK / WORLD_SIZE in the environment it is the launcher: it reads the rack
// inventory, builds the rank plan and starts one copy of itself per selected GPU on this host
// (the job that mpirun + rankfile do for the reference project, scripts/run_mnnvl_sharp.sh:252-263).
// Started with them (by its own launcher, by torchrun, or by any other process manager) it is
// one rank. Exit codes as in the reference's main (src/main.cc:491-505): 0 ok, 2 result check
// failed, 1 error; errors are printed as "rank R error: ...".
#include <unistd.h>

#include <cstdlib>
#include <exception>
#include <iostream>
#include <memory>
#include <string>
#include <vector>

#include "msharp/bootstrap.h"
#include "msharp/config.h"
#include "msharp/driver_api.h"
#include "msharp/rack.h"
#include "msharp/runner.h"

namespace {

bool launched_as_rank() {
  const char* rank = std::getenv("RANK");
  const char* world = std::getenv("WORLD_SIZE");
  return rank != nullptr && *rank != '\0' && world != nullptr && *world != '\0';
}

std::string self_path(const char* argv0) {
  char buf[4096];
  const ssize_t n = readlink("/proc/self/exe", buf, sizeof(buf) - 1);
  if (n > 0) {
    buf[n] = '\0';
    return buf;
  }
  return argv0;
}

}  // namespace

int main(int argc, char** argv) {
  int rank = 0;
  if (const char* r = std::getenv("RANK"); r != nullptr) {
    rank = std::atoi(r);
  }
  std::unique_ptr<msharp::Bootstrap> comm;
  try {
    const msharp::Config cfg = msharp::parse_config(argc, argv);
    if (cfg.cpu_only) {
      return msharp::run_cpu_only(cfg, std::cout);
    }
    if (!launched_as_rank()) {
      const msharp::RackConfig rack = msharp::RackConfig::load(cfg.rack_config_path);
      const int world = cfg.rank_count.value_or(static_cast<int>(rack.available_rank_count()));
      msharp::build_rank_plan(rack, world, cfg.rank_selection);  // fail early on a bad plan
      std::vector<std::string> args;
      args.push_back(self_path(argv[0]));
      for (int i = 1; i < argc; ++i) {
        args.emplace_back(argv[i]);
      }
      if (!cfg.rank_count) {
        args.emplace_back("--rank-count");
        args.emplace_back(std::to_string(world));
      }
      const std::string session = cfg.session.empty() ? "pid" + std::to_string(getpid()) : cfg.session;
      return msharp::spawn_local_ranks(args, world, session);
    }
    msharp::BootstrapOptions opt = msharp::Bootstrap::options_from_env();
    if (!cfg.session.empty()) {
      opt.session = cfg.session;
    }
    comm = msharp::Bootstrap::connect(opt);
    return msharp::run_rank(cfg, *comm, msharp::real_driver(), std::cout);
  } catch (const std::exception& ex) {
    std::cerr << "rank " << rank << " error: " << ex.what() << "\n";
    if (comm) {
      comm->abort(ex.what());
    }
    return 1;
  }
}

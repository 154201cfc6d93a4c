#include <signal.h>
#include <sys/wait.h>
#include <unistd.h>

#include <cerrno>
#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "msharp/runner.h"

namespace msharp {

int spawn_local_ranks(const std::vector<std::string>& argv, int world, const std::string& session) {
  std::vector<int> all;
  for (int rank = 0; rank < world; ++rank) {
    all.push_back(rank);
  }
  return spawn_host_ranks(argv, world, session, all, "");
}

int spawn_host_ranks(const std::vector<std::string>& argv, int world, const std::string& session,
                     const std::vector<int>& global_ranks, const std::string& hub_address) {
  if (argv.empty() || world <= 0 || global_ranks.empty()) {
    throw std::runtime_error("spawn: nothing to run");
  }
  std::vector<pid_t> children;
  for (std::size_t local = 0; local < global_ranks.size(); ++local) {
    const int rank = global_ranks[local];
    const pid_t pid = fork();
    if (pid < 0) {
      const std::string why = std::strerror(errno);
      for (pid_t c : children) {
        kill(c, SIGTERM);
      }
      throw std::runtime_error("spawn: fork failed: " + why);
    }
    if (pid == 0) {
      setenv("RANK", std::to_string(rank).c_str(), 1);
      setenv("LOCAL_RANK", std::to_string(local).c_str(), 1);
      setenv("WORLD_SIZE", std::to_string(world).c_str(), 1);
      setenv("MSHARP_SESSION", session.c_str(), 1);
      if (!hub_address.empty()) {
        setenv("MSHARP_HUB_ADDR", hub_address.c_str(), 1);
      }
      std::vector<char*> args;
      for (const auto& a : argv) {
        args.push_back(const_cast<char*>(a.c_str()));
      }
      args.push_back(nullptr);
      execv(args[0], args.data());
      std::fprintf(stderr, "spawn: exec %s failed: %s\n", args[0], std::strerror(errno));
      _exit(127);
    }
    children.push_back(pid);
  }
  int result = 0;
  std::size_t alive = children.size();
  while (alive > 0) {
    int status = 0;
    const pid_t done = waitpid(-1, &status, 0);
    if (done < 0) {
      if (errno == EINTR) {
        continue;
      }
      break;
    }
    bool ours = false;
    for (pid_t& c : children) {
      if (c == done) {
        c = -1;
        ours = true;
      }
    }
    if (!ours) {
      continue;
    }
    --alive;
    const int code = WIFEXITED(status) ? WEXITSTATUS(status) : 128 + (WIFSIGNALED(status) ? WTERMSIG(status) : 0);
    if (code != 0 && result == 0) {
      result = code;
      // The job is lost; the remaining ranks would only run into their bootstrap deadline.
      // Give them a moment to notice through the control plane and tear down in order, then end them.
      for (int waited = 0; waited < 50 && alive > 0; ++waited) {
        int st = 0;
        const pid_t more = waitpid(-1, &st, WNOHANG);
        if (more > 0) {
          for (pid_t& c : children) {
            if (c == more) {
              c = -1;
              --alive;
            }
          }
        } else {
          usleep(100000);
        }
      }
      for (pid_t c : children) {
        if (c > 0) {
          kill(c, SIGTERM);
        }
      }
    }
  }
  return result;
}

}  // namespace msharp

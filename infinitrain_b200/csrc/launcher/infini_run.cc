// infini_run: spawn one training process per local rank with the rendezvous environment set.
//
//   infini_run --nnodes=1 --nproc_per_node=8 --node_rank=0 --rdzv_endpoint=127.0.0.1:29500 -- prog args...
//
// Same role and flags as the reference launcher (tools/infini_run/infini_run.cc:11-58), which forks
// nproc_per_node children, exports NNODES / NPROC_PER_NODE / NODE_RANK / GLOBAL_PROC_RANK /
// LOCAL_PROC_RANK / PROC_WORLD_SIZE / MASTER_ADDR / MASTER_PORT and execvp()s the program.  This
// launcher additionally exports torchrun's names (RANK, LOCAL_RANK, WORLD_SIZE, LOCAL_WORLD_SIZE)
// because rendezvous here goes through torch.distributed's TCP store, and it supervises the
// children: when one exits with an error the others are terminated and the exit code is returned.
// With --max_restarts=N a failed attempt is followed by a new one (at most N times): the same program is started
// again on every local rank with ITB_RESTART_COUNT=<attempt> in its environment and the rendezvous port moved up by
// the attempt number (so that no rank of the new attempt meets a leftover of the old one); the trainers take
// ITB_RESTART_COUNT > 0 as "resume from the newest checkpoint under --save".  On several nodes every node's
// launcher restarts its own ranks; the attempts line up because a failure ends the ranks of every node.
#include <signal.h>
#include <sys/types.h>
#include <sys/wait.h>
#include <unistd.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

static bool flag(const char* arg, const char* name, std::string* out) {
  const size_t n = strlen(name);
  if (strncmp(arg, name, n) == 0 && arg[n] == '=') {
    *out = arg + n + 1;
    return true;
  }
  return false;
}

int main(int argc, char** argv) {
  std::string nnodes = "1", nproc = "1", node_rank = "0", rdzv = "127.0.0.1:29500", max_restarts = "0";
  int i = 1;
  for (; i < argc; ++i) {
    if (strcmp(argv[i], "--") == 0) { ++i; break; }
    if (flag(argv[i], "--nnodes", &nnodes) || flag(argv[i], "--nproc_per_node", &nproc) ||
        flag(argv[i], "--node_rank", &node_rank) || flag(argv[i], "--rdzv_endpoint", &rdzv) ||
        flag(argv[i], "--max_restarts", &max_restarts))
      continue;
    if (argv[i][0] != '-') break;   // first non-flag token starts the program
    fprintf(stderr, "infini_run: unknown flag %s\n", argv[i]);
    return 2;
  }
  if (i >= argc) {
    fprintf(stderr,
            "usage: infini_run [--nnodes=N] [--nproc_per_node=N] [--node_rank=R] "
            "[--rdzv_endpoint=host:port] [--max_restarts=N] [--] program [args...]\n");
    return 2;
  }
  const int n_nodes = atoi(nnodes.c_str()), n_proc = atoi(nproc.c_str()), nrank = atoi(node_rank.c_str());
  if (n_nodes < 1 || n_proc < 1 || nrank < 0 || nrank >= n_nodes) {
    fprintf(stderr, "infini_run: invalid topology\n");
    return 2;
  }
  std::string addr = rdzv, port = "29500";
  const size_t colon = rdzv.rfind(':');
  if (colon != std::string::npos) {
    addr = rdzv.substr(0, colon);
    port = rdzv.substr(colon + 1);
  }
  const int world = n_nodes * n_proc;
  const int restarts = atoi(max_restarts.c_str());
  if (restarts < 0) {
    fprintf(stderr, "infini_run: --max_restarts must not be negative\n");
    return 2;
  }
  int rc = 0;
  for (int attempt = 0; attempt <= restarts; ++attempt) {
    const std::string attempt_port = std::to_string(atoi(port.c_str()) + attempt);
    std::vector<pid_t> kids;
    for (int local = 0; local < n_proc; ++local) {
      pid_t pid = fork();
      if (pid < 0) { perror("fork"); return 1; }
      if (pid == 0) {
        const int global = nrank * n_proc + local;
        auto set = [](const char* k, const std::string& v) { setenv(k, v.c_str(), 1); };
        set("NNODES", nnodes);
        set("NPROC_PER_NODE", nproc);
        set("NODE_RANK", node_rank);
        set("GLOBAL_PROC_RANK", std::to_string(global));
        set("LOCAL_PROC_RANK", std::to_string(local));
        set("PROC_WORLD_SIZE", std::to_string(world));
        set("MASTER_ADDR", addr);
        set("MASTER_PORT", attempt_port);
        set("RANK", std::to_string(global));
        set("LOCAL_RANK", std::to_string(local));
        set("WORLD_SIZE", std::to_string(world));
        set("LOCAL_WORLD_SIZE", nproc);
        set("ITB_RESTART_COUNT", std::to_string(attempt));
        execvp(argv[i], argv + i);
        perror("execvp");
        _exit(127);
      }
      kids.push_back(pid);
    }
    rc = 0;
    size_t alive = kids.size();
    while (alive > 0) {
      int status = 0;
      pid_t done = wait(&status);
      if (done < 0) break;
      --alive;
      int code = WIFEXITED(status) ? WEXITSTATUS(status) : 128 + (WIFSIGNALED(status) ? WTERMSIG(status) : 0);
      if (code != 0 && rc == 0) {
        rc = code;
        for (pid_t k : kids)
          if (k != done) kill(k, SIGTERM);   // exact PIDs of our own children only
      }
    }
    if (rc == 0) return 0;
    if (attempt < restarts)
      fprintf(stderr, "infini_run: attempt %d ended with exit code %d; restarting (%d of %d)\n", attempt, rc, attempt + 1, restarts);
  }
  return rc;
}

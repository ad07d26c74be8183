/* shimrun -n <ranks> <program> [args...]: start the ranks of a program built against the
 * shared-memory MPI subset (mpi.h beside this file).  Creates the file the ranks map, starts one
 * process per rank with MPISHIM_FILE / MPISHIM_RANK / MPISHIM_SIZE set, waits for all of them and
 * returns the first non-zero exit status.  Baseline tooling. */
#define _GNU_SOURCE
#include <fcntl.h>
#include <signal.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/stat.h>
#include <sys/wait.h>
#include <unistd.h>

#define SHIM_RING_BYTES (2u << 20)
#define SHIM_COLL_CHUNK (4u << 20)

static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

int main(int argc, char** argv) {
  if (argc < 4 || strcmp(argv[1], "-n") != 0) {
    fprintf(stderr, "usage: %s -n <ranks> <program> [args...]\n", argv[0]);
    return 2;
  }
  const int n = atoi(argv[2]);
  if (n < 1 || n > 16) { fprintf(stderr, "shimrun: 1..16 ranks\n"); return 2; }
  /* generous upper bound of the layout in mpi_shim.c: header page, staging area, one ring per ordered pair */
  const size_t ring = align_up(SHIM_RING_BYTES + 4096, 4096);
  const size_t bytes = 8192 + (size_t)(n + 1) * SHIM_COLL_CHUNK + (size_t)n * n * ring;
  char path[256];
  struct stat st;
  snprintf(path, sizeof(path), "%s/mpishim_%d_XXXXXX", stat("/dev/shm", &st) == 0 ? "/dev/shm" : "/tmp", (int)getpid());
  int fd = mkstemp(path);
  if (fd < 0 || ftruncate(fd, (off_t)bytes) != 0) { perror("shimrun: shared file"); return 1; }
  close(fd);
  pid_t pids[16];
  for (int r = 0; r < n; ++r) {
    pids[r] = fork();
    if (pids[r] == 0) {
      char buf[32];
      setenv("MPISHIM_FILE", path, 1);
      snprintf(buf, sizeof(buf), "%d", r); setenv("MPISHIM_RANK", buf, 1);
      snprintf(buf, sizeof(buf), "%d", n); setenv("MPISHIM_SIZE", buf, 1);
      execvp(argv[3], argv + 3);
      perror("shimrun: exec");
      _exit(127);
    }
  }
  int rc = 0;
  for (int r = 0; r < n; ++r) {
    int status = 0;
    waitpid(pids[r], &status, 0);
    int code = WIFEXITED(status) ? WEXITSTATUS(status) : 128 + WTERMSIG(status);
    if (code != 0 && rc == 0) {
      rc = code;
      for (int q = 0; q < n; ++q) if (q != r) kill(pids[q], SIGTERM);   /* the ranks this launcher started */
    }
  }
  unlink(path);
  return rc;
}

/* The C interface from plain C: inventory and plan, then a communicator and a symmetric buffer.
 *
 *   cc -I csrc/include examples/c_api_symmetric_memory.c -L mnnvl_sharp_b200/_C -lmsharp -o c_api_example
 *   ./c_api_example            # host-memory driver stand-in: runs on any machine
 *   ./c_api_example real       # the GPU of ordinal 0
 *
 * One process is a world of one rank, which is enough to show the calls and their error
 * convention (0 / non-null on success, msharp_last_error() otherwise). With several ranks the
 * same calls are collective over the control plane returned by msharp_bootstrap_connect.
 */
#include <stdio.h>
#include <string.h>

#include "msharp/c_api.h"

static int fail(const char* what) {
  fprintf(stderr, "%s: %s\n", what, msharp_last_error());
  return 1;
}

int main(int argc, char** argv) {
  const int use_fake_driver = !(argc > 1 && strcmp(argv[1], "real") == 0);
  const char* yaml =
      "rack:\n"
      "  - tray-a:\n      - hostname: 10.0.0.11\n      - device: [0, 1, 2, 3]\n"
      "  - tray-b:\n      - hostname: 10.0.0.12\n      - device: [0, 1, 2, 3]\n";
  const char* plan = msharp_plan_from_yaml(yaml, 4, "balanced");
  if (plan == NULL) {
    return fail("plan");
  }
  printf("libmsharp %s\nbalanced plan for 4 ranks: %s\n", msharp_version(), plan);
  if (msharp_plan_from_yaml(yaml, 9, "balanced") != NULL) {
    fprintf(stderr, "a plan for more ranks than devices was accepted\n");
    return 1;
  }
  printf("asking for 9 ranks is refused: %s\n", msharp_last_error());

  if (use_fake_driver) {
    msharp_fake_driver_reset(8);
  }
  void* boot = msharp_bootstrap_connect(0, 1, "c-example", 10000);
  if (boot == NULL) {
    return fail("bootstrap");
  }
  void* comm = msharp_comm_create(boot, 0, 2000, use_fake_driver, 0);
  if (comm == NULL) {
    return fail("communicator");
  }
  printf("communicator: %s\n", msharp_comm_info(comm));
  void* buf = msharp_symm_alloc(comm, (size_t)3 << 20, 0, 1);
  if (buf == NULL) {
    return fail("symmetric allocation");
  }
  printf("buffer: %s\n", msharp_symm_info(buf));

  unsigned char out[16];
  unsigned char in[16];
  for (int i = 0; i < 16; ++i) {
    out[i] = (unsigned char)(0xa0 + i);
  }
  if (msharp_symm_copy_from_host(buf, 0, 4096, out, sizeof(out)) != 0 ||
      msharp_symm_copy_to_host(buf, in, 0, 4096, sizeof(in)) != 0) {
    return fail("copy");
  }
  if (memcmp(in, out, sizeof(in)) != 0) {
    fprintf(stderr, "read back different bytes\n");
    return 1;
  }
  if (msharp_symm_copy_to_host(buf, in, 0, ((size_t)3 << 20) + (1 << 20), 16) == 0) {
    fprintf(stderr, "a read beyond the allocation was accepted\n");
    return 1;
  }
  printf("out-of-range read is refused: %s\n", msharp_last_error());

  if (msharp_symm_free(buf) != 0 || msharp_comm_destroy(comm) != 0) {
    return fail("teardown");
  }
  msharp_bootstrap_destroy(boot);
  printf("ok\n");
  return 0;
}

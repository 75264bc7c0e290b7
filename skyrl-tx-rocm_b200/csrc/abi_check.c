/* Plain-C (C11) consumer of the C ABI: proves that the public header compiles as C, that the
 * compile-time layout checks hold for a C compiler too, and that the size queries link and run
 * without a GPU.  Built by build.py next to the library; run by the CPU test-suite. */
#include <stdio.h>
#include <string.h>

#include "../../include/skyrl_w8a8_sm100.h"

int main(void) {
  SkyrlW8A8LinearArgs lin;
  SkyrlW8A8MlpArgs mlp;
  memset(&lin, 0, sizeof lin);
  memset(&mlp, 0, sizeof mlp);
  lin.struct_size = (uint32_t)sizeof lin;
  mlp.struct_size = (uint32_t)sizeof mlp;
  if (skyrl_w8a8_abi_version() != SKYRL_W8A8_ABI_VERSION) {
    fprintf(stderr, "ABI version mismatch\n");
    return 1;
  }
  const size_t lin_ws = skyrl_w8a8_linear_workspace_bytes(256, 3072, 1024, 1);
  const size_t mlp_ws = skyrl_w8a8_mlp_workspace_bytes(16384, 5120, 25600, 16);
  const size_t none = skyrl_w8a8_linear_workspace_bytes(0, 3072, 1024, 1);
  /* a call without buffers is refused with a message, never a crash */
  const int rc = skyrl_w8a8_lora_forward_sm100_v1(&lin, NULL);
  printf("abi=%d linear_ws=%zu mlp_ws=%zu empty=%zu rc=%d err=\"%s\"\n", skyrl_w8a8_abi_version(), lin_ws, mlp_ws, none, rc,
         skyrl_w8a8_last_error());
  return (lin_ws > 0 && mlp_ws > lin_ws && none == 0 && rc == SKYRL_ERR_INVALID_ARGUMENT) ? 0 : 2;
}

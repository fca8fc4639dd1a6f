// CPU oracle, part 3: FLASH_ATTN_EXT.  TEST INFRASTRUCTURE ONLY (see oracle.h).
#include "oracle.h"
extern "C" int orc_flash_attn_ext(const OrcFlashArgs *) { return -1; }

#include "health/consistency.h"
#include <cstdlib>
#include <cstring>
namespace hcclb {
uint32_t crc32(const void *data, size_t len, uint32_t seed)
{
    struct Table {
        uint32_t v[256];
        Table()
        {
            for (uint32_t i = 0; i < 256; ++i) {
                uint32_t c = i;
                for (int k = 0; k < 8; ++k) c = (c & 1) ? (0xEDB88320u ^ (c >> 1)) : (c >> 1);
                v[i] = c;
            }
        }
    };
    static const Table tab;  // built once, also when several ranks of one process start together
    const uint32_t *table = tab.v;
    uint32_t c = ~seed;
    const uint8_t *p = (const uint8_t *)data;
    for (size_t i = 0; i < len; ++i) c = table[(c ^ p[i]) & 0xff] ^ (c >> 8);
    return ~c;
}
bool consistency_enabled()
{
    const char *e = getenv("HCCL_CONSISTENCY_CHECK");
    return !(e && strcmp(e, "0") == 0);
}
}  // namespace hcclb

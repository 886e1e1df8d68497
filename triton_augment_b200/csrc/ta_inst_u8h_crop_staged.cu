#include "ta_tables.cuh"
namespace ta {
const KernelTable &table_u8h_crop_staged() { return make_table<__half, 3, uint8_t>(); }
}

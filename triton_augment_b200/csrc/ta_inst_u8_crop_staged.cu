#include "ta_tables.cuh"
namespace ta {
const KernelTable &table_u8_crop_staged() { return make_table<float, 3, uint8_t>(); }
}

#include "ta_tables.cuh"
namespace ta {
const KernelTable &table_u8_bilinear_mix() { return make_table<float, 4, uint8_t>(); }
}

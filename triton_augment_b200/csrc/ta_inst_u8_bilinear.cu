#include "ta_tables.cuh"
namespace ta {
const KernelTable &table_u8_bilinear() { return make_table<float, 2, uint8_t>(); }
}

#include "ta_tables.cuh"
namespace ta {
const KernelTable &table_u8h_bilinear() { return make_table<__half, 2, uint8_t>(); }
}

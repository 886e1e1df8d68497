#include "ta_tables.cuh"
namespace ta {
const KernelTable &table_u8_nearest() { return make_table<float, 1, uint8_t>(); }
}

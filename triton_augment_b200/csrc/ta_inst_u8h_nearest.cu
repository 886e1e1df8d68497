#include "ta_tables.cuh"
namespace ta {
const KernelTable &table_u8h_nearest() { return make_table<__half, 1, uint8_t>(); }
}

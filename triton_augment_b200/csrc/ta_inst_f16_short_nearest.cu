#include "ta_tables.cuh"
namespace ta {
const KernelTable &table_f16_short_nearest() { return make_table<__half, 1, __half, kTileHShort>(); }
}

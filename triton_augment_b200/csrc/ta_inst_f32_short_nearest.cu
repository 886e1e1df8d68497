#include "ta_tables.cuh"
namespace ta {
const KernelTable &table_f32_short_nearest() { return make_table<float, 1, float, kTileHShort>(); }
}

#include "ta_tables.cuh"
namespace ta {
const KernelTable &table_f32_short_bilinear_mix() { return make_table<float, 4, float, kTileHShort>(); }
}

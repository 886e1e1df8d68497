#include "ta_tables.cuh"
namespace ta {
const KernelTable &table_f32_short_bilinear() { return make_table<float, 2, float, kTileHShort>(); }
}

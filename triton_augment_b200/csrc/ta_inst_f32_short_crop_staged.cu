#include "ta_tables.cuh"
namespace ta {
const KernelTable &table_f32_short_crop_staged() { return make_table<float, 3, float, kTileHShort>(); }
}

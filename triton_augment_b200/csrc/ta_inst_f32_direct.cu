#include "ta_tables.cuh"
namespace ta {
const KernelTable &table_f32_direct() { return make_table<float, 0>(); }
}

#include "ta_tables.cuh"
namespace ta {
const KernelTable &table_f32_nearest() { return make_table<float, 1>(); }
}

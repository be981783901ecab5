// Helpers shared between the NUMA entry points and the correction worker pool.
#pragma once
#include <vector>

namespace jf {
bool node_cpus(int node, std::vector<int>* cpus);   // processors of a node from sysfs; false if unknown
int worker_node();                                   // node the correction workers are confined to, -1 = none
bool pin_this_thread_to_node(int node);
}  // namespace jf

// Definition of the opaque cavs_sched handle, shared by the C ABI of the scheduler and
// the engines that consume a loaded schedule.
#ifndef CAVS_B200_HOST_SCHED_HANDLE_H_
#define CAVS_B200_HOST_SCHED_HANDLE_H_
#include "host/schedule.h"
struct cavs_sched {
  cavs_b200::LevelSchedule impl;
  bool loaded = false;
};
#endif

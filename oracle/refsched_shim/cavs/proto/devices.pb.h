// Stand-in for the protobuf-generated device enum.  TEST INFRASTRUCTURE.
#ifndef ORACLE_SHIM_CAVS_PROTO_DEVICES_PB_H_
#define ORACLE_SHIM_CAVS_PROTO_DEVICES_PB_H_
enum DeviceType { CPU = 0, GPU = 1 };
#endif

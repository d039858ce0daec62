// Folded into op_def.pb.h (the protobuf-free message classes).
#include "cavs/proto/op_def.pb.h"

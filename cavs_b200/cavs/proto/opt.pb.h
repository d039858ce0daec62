// Optimisation switches of Session(int opt), same values as cavs/proto/opt.proto:3-8.
#ifndef CAVS_PROTO_OPT_PB_H_
#define CAVS_PROTO_OPT_PB_H_
enum OptimizationType { OPT_NONE = 0, OPT_FUSION = 1, OPT_BATCHING = 2, OPT_STREAMMING = 4 };
#endif

// Attribute and naming helpers, same signatures as cavs/util/op_util.h:6-24.
#ifndef CAVS_UTIL_OP_UTIL_H_
#define CAVS_UTIL_OP_UTIL_H_

#include <string>
#include <vector>

#include "cavs/proto/op_def.pb.h"

template <typename T> T GetSingleArg(const OpDef& op_def, const std::string& key);
template <typename T> T GetSingleArg(const OpDef& op_def, const std::string& key, T value);
template <typename T> std::vector<T> GetListArg(const OpDef& op_def, const std::string& key);

std::string GetGradientName(const std::string& op);   // "X" -> "X_grad" (cavs/util/op_util.cc:9-17)
std::string GetOriginName(const std::string& op);
const char* DeviceTypeToString(DeviceType type);
size_t GetHash(const OpDef& op_def);
bool IsGradientName(const std::string& edge);
#endif

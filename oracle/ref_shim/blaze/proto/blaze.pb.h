// Hand-written stand-in for the protobuf-generated blaze/proto/blaze.pb.h.
//
// TEST INFRASTRUCTURE ONLY. The reference's store sources only need the
// DataType enumerators from the generated header; building protoc just for
// them is not worth it, so this header restates the enum with the numeric
// values of blaze/blaze/proto/blaze.proto:6-20.
#pragma once
namespace blaze {
enum DataType {
  kFloat = 1,
  kInt32 = 2,
  kByte = 3,
  kString = 4,
  kBool = 5,
  kUInt8 = 6,
  kInt8 = 7,
  kUInt16 = 8,
  kInt16 = 9,
  kInt64 = 10,
  kFloat16 = 12,
  kDouble = 13,
};
}  // namespace blaze

#!/bin/bash
# TEST INFRASTRUCTURE ONLY - nothing here ships.
# Builds oracle/_ref/libblaze_cpu.so: the reference's own CPU implementation of the dense operators, the
# Embedding operator, the sparse store, Workspace and Net, compiled unmodified from the sources where they lie in
# a reference checkout, together with oracle/ref_dense_glue.cc and oracle/ref_glue.cc (C interfaces for ctypes).
# Outputs go under oracle/_ref/ only. The library is a superset of _ref/libqed_ref.so (oracle/Makefile); a process
# loads one of the two, never both: they would register the reference's sparse puller twice.
#
#   usage: oracle/build_ref_dense.sh <root of the reference checkout> [jobs]
#
# Steps (the reference's own build system is not run):
#   1. the vendored protobuf 3.6.0 runtime and a protoc with the C++ generator only, by hand from
#      blaze/thirdparty/protobuf/protobuf-3.6.0/src;
#   2. blaze.pb / embedding.pb / fusion_pattern.pb generated from blaze/blaze/proto/*.proto;
#   3. every .cc under blaze/blaze/{common,store,math,operator,graph,optimizer,scheduler,batching} without
#      USE_CUDA / USE_MKL, with the headers GCC 13 no longer includes transitively forced in and
#      oracle/ref_shim/cblas.h standing in for the OpenBLAS header.
set -e
REF=${1:?reference checkout}
JOBS=${2:-8}
HERE=$(cd "$(dirname "$0")" && pwd)
OUT=$HERE/_ref
B=$OUT/build
PB=$REF/blaze/thirdparty/protobuf/protobuf-3.6.0/src
BLZ=$REF/blaze
mkdir -p $B/pb $B/protoc $B/gen/blaze $B/blaze

cc_pb() {   # source (relative to $PB) -> object
  local o=$B/pb/$(echo $1 | tr '/' '_').o
  [ -f $o ] || g++ -std=c++14 -O1 -fPIC -w -DHAVE_PTHREAD -I$PB -c $PB/$1 -o $o
}
export -f cc_pb; export B PB

RUNTIME="arena.cc arenastring.cc extension_set.cc generated_message_table_driven_lite.cc generated_message_util.cc
implicit_weak_message.cc io/coded_stream.cc io/zero_copy_stream.cc io/zero_copy_stream_impl_lite.cc message_lite.cc
repeated_field.cc stubs/bytestream.cc stubs/common.cc stubs/int128.cc stubs/status.cc stubs/statusor.cc
stubs/stringpiece.cc stubs/stringprintf.cc stubs/structurally_valid.cc stubs/strutil.cc stubs/time.cc wire_format_lite.cc
any.cc any.pb.cc api.pb.cc compiler/importer.cc compiler/parser.cc descriptor.cc descriptor.pb.cc descriptor_database.cc
duration.pb.cc dynamic_message.cc empty.pb.cc extension_set_heavy.cc field_mask.pb.cc generated_message_reflection.cc
generated_message_table_driven.cc io/gzip_stream.cc io/printer.cc io/strtod.cc io/tokenizer.cc io/zero_copy_stream_impl.cc
map_field.cc message.cc reflection_ops.cc service.cc source_context.pb.cc struct.pb.cc stubs/mathlimits.cc
stubs/substitute.cc text_format.cc timestamp.pb.cc type.pb.cc unknown_field_set.cc wire_format.cc wrappers.pb.cc"
PROTOC="compiler/code_generator.cc compiler/command_line_interface.cc compiler/plugin.cc compiler/plugin.pb.cc
compiler/subprocess.cc compiler/zip_writer.cc compiler/cpp/cpp_enum.cc compiler/cpp/cpp_enum_field.cc
compiler/cpp/cpp_extension.cc compiler/cpp/cpp_field.cc compiler/cpp/cpp_file.cc compiler/cpp/cpp_generator.cc
compiler/cpp/cpp_helpers.cc compiler/cpp/cpp_map_field.cc compiler/cpp/cpp_message.cc compiler/cpp/cpp_message_field.cc
compiler/cpp/cpp_padding_optimizer.cc compiler/cpp/cpp_primitive_field.cc compiler/cpp/cpp_service.cc
compiler/cpp/cpp_string_field.cc"

echo "[1/4] protobuf runtime and protoc"
for f in $RUNTIME $PROTOC; do echo google/protobuf/$f; done | xargs -P $JOBS -I{} bash -c 'cc_pb {}'
if [ ! -x $B/protoc/protoc ]; then
  cat > $B/protoc/main.cc <<'EOC'
#include <google/protobuf/compiler/command_line_interface.h>
#include <google/protobuf/compiler/cpp/cpp_generator.h>
int main(int argc, char* argv[]) {
  google::protobuf::compiler::CommandLineInterface cli;
  google::protobuf::compiler::cpp::CppGenerator cpp;
  cli.RegisterGenerator("--cpp_out", "--cpp_opt", &cpp, "C++ header and source");
  return cli.Run(argc, argv);
}
EOC
  g++ -std=c++14 -O1 -w -DHAVE_PTHREAD -I$PB $B/protoc/main.cc $B/pb/*.o -o $B/protoc/protoc -lpthread
fi

echo "[2/4] generated protocol headers"
for p in blaze embedding fusion_pattern; do
  [ -f $B/gen/blaze/proto/$p.pb.cc ] || $B/protoc/protoc --cpp_out=$B/gen/blaze -I$BLZ/blaze $BLZ/blaze/proto/$p.proto
done

echo "[3/4] reference CPU sources"
FORCED="-include functional -include cstdint -include cstring -include numeric -include string -include cmath -include memory -include limits"
# the reference's own flags (blaze/CMakeLists.txt:78), warnings off
FLAGS="-O2 -DNDEBUG -std=c++11 -fPIC -ftree-vectorize -w -mavx -mavx2 -mf16c -fopenmp -DHAVE_PTHREAD $FORCED -I$B/gen -I$B/gen/blaze -I$HERE/ref_shim -I$BLZ -I$PB"
cc_blz() {
  local o=$B/blaze/$(echo ${1#$BLZ/} | tr '/' '_').o
  [ -f $o ] || g++ $FLAGS -c $1 -o $o || echo "FAILED $1" >> $B/blaze/failed.txt
}
export -f cc_blz; export FLAGS BLZ
rm -f $B/blaze/failed.txt
( find $BLZ/blaze/common $BLZ/blaze/store $BLZ/blaze/math $BLZ/blaze/operator $BLZ/blaze/graph $BLZ/blaze/optimizer \
       $BLZ/blaze/scheduler $BLZ/blaze/batching -name '*.cc'; ls $B/gen/blaze/proto/*.pb.cc ) | \
  xargs -P $JOBS -I{} bash -c 'cc_blz {}'
if [ -f $B/blaze/failed.txt ]; then cat $B/blaze/failed.txt; exit 1; fi

echo "[4/4] link"
RT_OBJS=$(for f in $RUNTIME; do echo $B/pb/$(echo google/protobuf/$f | tr '/' '_').o; done)
g++ -O2 -DNDEBUG -std=c++11 -fPIC -ftree-vectorize -w -mavx -mavx2 -mf16c -shared -fopenmp $FORCED -I$B/gen -I$HERE/ref_shim -I$BLZ -I$PB \
    $HERE/ref_dense_glue.cc $HERE/ref_glue.cc $B/blaze/*.o $RT_OBJS -o $OUT/libblaze_cpu.so -lpthread -ldl
echo "built $OUT/libblaze_cpu.so"

"""A C++ consumer of the link-level boundary: a translation unit that is compiled against
include/aicf/backends/cuda/registry/*.hpp with plain g++, links libaicf_b200.so, registers an out-of-tree kernel
variant through KernelRegistry::register_kernel and has it chosen by both dispatch paths (by id and by priority),
exactly what a maintainer of the reference does when adding an op outside the library
(reference: src/backends/cuda/registry/registry.cpp:76-115 register_kernel, :16-64 by-id path, :144-195 priority
path). The variant's launch only sets host flags, so the test needs no GPU."""
import os
import shutil
import subprocess
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parents[1]
LIB_DIR = REPO / "ai-compiler-framework_b200" / "lib"

SOURCE = r"""
#include <cstdio>
#include <cstring>
#include <vector>

#include "aicf/backends/cuda/registry/attr_blob.hpp"
#include "aicf/backends/cuda/registry/dispatch.hpp"
#include "aicf/backends/cuda/registry/registry.hpp"

using namespace aicf::cuda;

static int g_launches = 0;
static uint32_t g_schema_seen = 0xdeadbeefu;
static const void* g_workspace_seen = reinterpret_cast<const void*>(1);
static int64_t g_rows_seen = -1;

// Takes exactly one int32 tensor of 12345 elements: nothing in the library ever sees such a call by accident.
static bool mine_supported(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void*) {
  return ni == 1 && no == 1 && in && out && in[0].dtype == DType::kI32 && in[0].rank() == 1 && in[0].shape[0] == 12345;
}
static Status mine_launch(const TensorDesc* in, int, TensorDesc*, int, const void* attr, void* ws, size_t, cudaStream_t) {
  ++g_launches;
  g_schema_seen = static_cast<const AttrBlob*>(attr)->schema_id;  // never null inside a variant
  g_workspace_seen = ws;
  g_rows_seen = in[0].shape[0];
  return Status::Ok;
}
static bool never_supported(const TensorDesc*, int, const TensorDesc*, int, const void*) { return false; }

static TensorDesc i32_vector(int64_t n) {
  TensorDesc t{};
  t.data = reinterpret_cast<void*>(0x1000);  // never dereferenced
  t.dtype = DType::kI32;
  t.r.rank = 1;
  t.shape[0] = n;
  t.stride[0] = 1;
  t.contiguous = true;
  return t;
}

#define EXPECT(cond)                                                   \
  do {                                                                 \
    if (!(cond)) { std::printf("FAIL line %d: %s\n", __LINE__, #cond); return 1; } \
  } while (0)

int main() {
  KernelVariant v{};
  v.name = "consumer_copy";
  v.kernel_id = "consumer_copy_i32_v0";
  v.priority = 1000;  // ahead of every built-in Copy variant
  v.launch = mine_launch;
  v.supported = mine_supported;
  KernelRegistry::instance().register_kernel(OpKind::Copy, v);

  KernelVariant refuses = v;  // same kind, higher priority, never takes a call: the dispatcher must move on
  refuses.kernel_id = "consumer_never_v0";
  refuses.priority = 2000;
  refuses.supported = never_supported;
  KernelRegistry::instance().register_kernel(OpKind::Copy, refuses);

  KernelVariant dup = v;  // the first registration of an id wins
  dup.priority = 5;
  KernelRegistry::instance().register_kernel(OpKind::Copy, dup);
  KernelVariant anonymous = v;  // ignored: a variant must carry an id
  anonymous.kernel_id = nullptr;
  KernelRegistry::instance().register_kernel(OpKind::Copy, anonymous);

  EXPECT(KernelRegistry::instance().find_by_id(OpKind::Copy, "consumer_copy_i32_v0") != nullptr);
  EXPECT(KernelRegistry::instance().find_by_id(OpKind::Copy, "consumer_copy_i32_v0")->priority == 1000);
  EXPECT(KernelRegistry::instance().find_by_id(OpKind::Gemm, "consumer_copy_i32_v0") == nullptr);

  TensorDesc in = i32_vector(12345), out = i32_vector(12345);

  // by id, without attrs: the variant sees an empty blob, not a null pointer
  EXPECT(dispatch_by_id_v0(OpKind::Copy, "consumer_copy_i32_v0", &in, 1, &out, 1, nullptr, nullptr) == Status::Ok);
  EXPECT(g_launches == 1 && g_schema_seen == 0u && g_workspace_seen == nullptr && g_rows_seen == 12345);

  // by id, with attrs
  const int32_t payload = 7;
  AttrBlob blob{};
  blob.schema_id = 0x54534554u;
  blob.bytes = 4;
  blob.data = &payload;
  EXPECT(dispatch_by_id_v0(OpKind::Copy, "consumer_copy_i32_v0", &in, 1, &out, 1, &blob, nullptr) == Status::Ok);
  EXPECT(g_launches == 2 && g_schema_seen == 0x54534554u);

  // by priority: the 2000-priority variant refuses, the 1000-priority one runs, the built-ins are never asked
  EXPECT(dispatch_v0(OpKind::Copy, &in, 1, &out, 1, nullptr, nullptr) == Status::Ok);
  EXPECT(g_launches == 3);

  // the status rules of the by-id path
  TensorDesc other = i32_vector(7);
  EXPECT(dispatch_by_id_v0(OpKind::Copy, "consumer_copy_i32_v0", &other, 1, &out, 1, nullptr, nullptr) == Status::InvalidArgument);
  EXPECT(dispatch_by_id_v0(OpKind::Copy, "consumer_never_v0", &in, 1, &out, 1, nullptr, nullptr) == Status::InvalidArgument);
  EXPECT(dispatch_by_id_v0(OpKind::Copy, "no_such_kernel_v0", &in, 1, &out, 1, nullptr, nullptr) == Status::NotImplemented);
  EXPECT(dispatch_by_id_v0(OpKind::Gemm, "consumer_copy_i32_v0", &in, 1, &out, 1, nullptr, nullptr) == Status::NotImplemented);
  EXPECT(dispatch_by_id_v0(OpKind::Copy, "", &in, 1, &out, 1, nullptr, nullptr) == Status::InvalidArgument);
  EXPECT(g_launches == 3);

  // a mandatory schema is enforced before supported() is asked
  KernelVariant strict = v;
  strict.kernel_id = "consumer_strict_v0";
  strict.expected_attr_schema_id = 0x54534554u;
  KernelRegistry::instance().register_kernel(OpKind::Copy, strict);
  EXPECT(dispatch_by_id_v0(OpKind::Copy, "consumer_strict_v0", &in, 1, &out, 1, nullptr, nullptr) == Status::InvalidArgument);
  EXPECT(dispatch_by_id_v0(OpKind::Copy, "consumer_strict_v0", &in, 1, &out, 1, &blob, nullptr) == Status::Ok);
  EXPECT(g_launches == 4);

  // the library's own kernels are still there, behind the out-of-tree ones
  std::vector<const KernelVariant*> all;
  KernelRegistry::instance().variants_snapshot(OpKind::Copy, all);
  EXPECT(all.size() >= 7);
  EXPECT(std::strcmp(all[0]->kernel_id, "consumer_never_v0") == 0 && std::strcmp(all[1]->kernel_id, "consumer_copy_i32_v0") == 0);
  EXPECT(KernelRegistry::instance().find_by_id(OpKind::Copy, "copy_f32_v0") != nullptr);
  for (size_t i = 1; i < all.size(); ++i) EXPECT(all[i - 1]->priority >= all[i]->priority);

  std::printf("CONSUMER_OK launches=%d\n", g_launches);
  return 0;
}
"""


def _cuda_include() -> Path:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return Path(nvcc).resolve().parents[1] / "include"


def test_out_of_tree_variant_registers_and_dispatches(tmp_path):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("g++ not available")
    assert (LIB_DIR / "libaicf_b200.so").exists(), "build the library first (python ai-compiler-framework_b200/build.py)"
    src, exe = tmp_path / "consumer.cpp", tmp_path / "consumer"
    src.write_text(SOURCE)
    cmd = [gxx, "-std=c++17", "-O1", f"-I{REPO / 'include'}", f"-I{_cuda_include()}", str(src), "-o", str(exe),
           f"-L{LIB_DIR}", "-laicf_b200", f"-Wl,-rpath,{LIB_DIR}"]
    built = subprocess.run(cmd, capture_output=True, text=True)
    assert built.returncode == 0, f"the consumer does not compile or link against the public headers:\n{built.stderr}"
    env = dict(os.environ, LD_LIBRARY_PATH=f"{LIB_DIR}:{os.environ.get('LD_LIBRARY_PATH', '')}")
    ran = subprocess.run([str(exe)], capture_output=True, text=True, env=env, timeout=120)
    assert ran.returncode == 0 and "CONSUMER_OK launches=4" in ran.stdout, ran.stdout + ran.stderr

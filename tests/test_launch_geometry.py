"""Host-side launch geometry of the row kernels and the streaming kernels, checked without a GPU: a small program
compiled with nvcc against csrc/kernels/row_pipeline.cuh (host code only; without a device the SM count falls back to
the B200's 148) walks every row length and checks the invariants the kernels rely on. Nothing here mirrors a reference
interface: the reference launches one block per row or a fixed 65535-block grid."""
import os
import shutil
import subprocess
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parents[1]
KERNELS = REPO / "ai-compiler-framework_b200" / "csrc" / "kernels"

SOURCE = r"""
#include <cstdio>
#include <cstdint>

#include "row_pipeline.cuh"

using namespace aicf::cuda;
using namespace aicf::cuda::rowk;

#define EXPECT(cond)                                                                       \
  do {                                                                                     \
    if (!(cond)) { std::printf("FAIL line %d: %s (n=%lld)\n", __LINE__, #cond, (long long)n); return 1; } \
  } while (0)

int main() {
  long long n = 0;
  // threads / packets per thread for every row length in packets, for both register budgets (fp32: 8, 16-bit: 4)
  for (int max_packets : {8, 4}) {
    for (n = 1; n <= 40000; ++n) {
      const RowCfg c = pick_row_cfg(n, max_packets);
      if (c.packets == 0) {  // the fallback: only for rows no block can hold
        EXPECT(n > 1024LL * max_packets);
        continue;
      }
      EXPECT(c.threads >= 32 && c.threads <= 1024 && (c.threads & (c.threads - 1)) == 0);
      EXPECT(c.packets == 1 || c.packets == 2 || c.packets == 4 || c.packets == 8);
      EXPECT(c.packets <= max_packets);
      EXPECT(static_cast<long long>(c.threads) * c.packets >= n);          // the block covers the row
      EXPECT(c.threads == 32 || static_cast<long long>(c.threads / 2) * 4 < n);  // and is no larger than it has to be
    }
  }
  // resident blocks estimate and the residency cap of softmax / cross-entropy
  for (int threads = 32; threads <= 1024; threads *= 2) {
    for (n = 64; n <= 200 * 1024; n += 1040) {
      const size_t smem = row_pipe_smem(n);
      EXPECT(smem >= static_cast<size_t>(n) + 16);
      const int est = row_pipe_blocks_per_sm(threads, smem);
      EXPECT(est >= 1 && est <= 32 && est * threads <= 2048);
      EXPECT(static_cast<size_t>(est) * (smem + 1024) <= 227 * 1024 || est == 1);
      const size_t capped = row_smem_capped_residency(smem, threads);
      EXPECT(capped >= smem && capped <= 227 * 1024 && capped % 16 == 0 || capped == smem);
      const size_t fit_before = (227 * 1024) / (smem + 1024), fit = (227 * 1024) / (capped + 1024);
      if (threads >= 128) {
        const size_t want = static_cast<size_t>(1024 / threads);
        EXPECT(fit * threads <= 1024);                                    // never more than 1024 threads resident
        EXPECT(fit >= (fit_before < want ? fit_before : want));           // and never fewer than the cap asks for
      } else {
        EXPECT(capped == smem);
      }
    }
  }
  // streaming grids: at least one block, never more than the work or the cap
  for (n = 0; n <= (1LL << 34); n = n * 3 + 1) {
    for (int per_sm : {1, 8, kStreamBlocksPerSm}) {
      const int g = streaming_grid(n, 256, per_sm);
      EXPECT(g >= 1 && g <= sm_count() * per_sm);
      EXPECT(n <= 0 || static_cast<long long>(g - 1) * 256 < n);
    }
  }
  // 16-bit kernels take the lean variant on an exact fit, fp32 kernels keep the checked one
  n = 0;
  EXPECT(use_full_rows(true, 2) && !use_full_rows(true, 4) && !use_full_rows(false, 2));
  std::printf("ok\n");
  return 0;
}
"""


@pytest.mark.skipif(shutil.which("nvcc") is None, reason="needs nvcc")
def test_row_and_streaming_launch_geometry(tmp_path):
    src = tmp_path / "geometry.cu"
    src.write_text(SOURCE)
    exe = tmp_path / "geometry"
    env = {k: v for k, v in os.environ.items() if not k.startswith("AICF_ROW") and k != "AICF_ROW_FULL"}
    build = subprocess.run(["nvcc", "-std=c++17", "-O1", "-I", str(KERNELS), "-I", str(REPO / "include"), "-o", str(exe), str(src)],
                           capture_output=True, text=True)
    assert build.returncode == 0, build.stderr[-3000:]
    run = subprocess.run([str(exe)], capture_output=True, text=True, env=env)
    assert run.returncode == 0 and run.stdout.strip().endswith("ok"), run.stdout[-2000:] + run.stderr[-2000:]

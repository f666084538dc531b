"""The C++ host header (reference names over the C ABI) compiles and links against the library."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SRC = r'''
#include "crucible_layers.hpp"
#include <cstdio>
int main() {
  crucible::Geometry g{2048, 16, 2, 32, 16};
  crucible::GdnArgs a{};
  a.R = 0;
  if (crucible::LaunchGdnCore(g, a) != CR_ERR_INVALID) return 1;          // contract violation, no device needed
  try { crucible::Check(crucible::LaunchGdnCore(g, a)); return 2; } catch (const std::runtime_error&) {}
  static_assert(crucible::QsaPoolOffset(33, 2) == 4096 + 64 + 1, "pool layout");
  static_assert(crucible::OutProjIndex(3, 17, 4096, 8, 1) == (size_t)(1 * 8 + 4) * 16 + 1, "packed layout");
  if (crucible::QsaPoolFloats(262144) != 2048u * 4096u) return 3;
  if (crucible::QsaScratchBytes(g, 1) != 16u * 32u * 258u * 4u) return 4;
  std::puts("ok");
  return 0;
}
'''


def test_host_header_compiles_and_links(tmp_path):
    import __graft_entry__ as ge
    ge.build()
    src = tmp_path / "host.cpp"
    src.write_text(SRC)
    exe = tmp_path / "host"
    pkg = os.path.join(ROOT, "crucible_strix_halo_b200")
    subprocess.check_call(["g++", "-std=c++17", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe),
                           "-L", pkg, "-lcrucible_attn", "-Wl,-rpath," + pkg])
    env = dict(os.environ)
    out = subprocess.run([str(exe)], capture_output=True, text=True, env=env)
    assert out.returncode == 0 and "ok" in out.stdout, (out.returncode, out.stdout, out.stderr)

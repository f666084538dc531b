"""The host-side state contracts (include/crucible_state.hpp: commit / replay ledger, verify-span rules, fixed-state
visit order and byte totals, cache sizes) pass the reference's CPU contract cases, compiled with g++ alone."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_state_contract_cases(tmp_path):
    exe = str(tmp_path / "state_contracts_test")
    src = os.path.join(ROOT, "tests", "state_contracts_test.cpp")
    cc = subprocess.run(["g++", "-std=c++17", "-O1", "-Wall", "-Wextra", "-Werror", "-fsanitize=undefined", "-fno-sanitize-recover",
                         "-I", os.path.join(ROOT, "include"), src, "-o", exe], capture_output=True, text=True)
    assert cc.returncode == 0, cc.stderr
    run = subprocess.run([exe], capture_output=True, text=True)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "state_contracts_test: ok" in run.stdout

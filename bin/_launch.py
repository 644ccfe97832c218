"""Shared by the launchers in this folder: builds libb200llm.so on first use (nvcc, in-tree) and calls the package's command line."""
import importlib
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(command):
    lib = os.path.join(ROOT, "llm-inference-engine_b200", "lib", "libb200llm.so")
    if not os.path.exists(lib):
        jobs = str(min(16, os.cpu_count() or 4))
        r = subprocess.run(["make", "-s", "-j" + jobs, "-C", os.path.join(ROOT, "llm-inference-engine_b200", "csrc")], stdout=sys.stderr)
        if r.returncode != 0:
            sys.exit("building libb200llm.so failed")
    sys.path.insert(0, ROOT)
    sys.dont_write_bytecode = True
    cli = importlib.import_module("llm-inference-engine_b200.cli")
    sys.exit(cli.main([command] + sys.argv[1:]))

"""Binding of the collective library, without a GPU: the communicator calls answer COMM_FAILED when the
named NCCL file does not load (no other copy is looked for), and bind whatever file is named."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PROBE = r'''
import os, sys
sys.path.insert(0, os.environ["SYN_ROOT"])
from synaptik_b200 import native
try:
    print("id", native.comm_unique_id().hex())
except native.NativeFailure as failure:
    print("status", failure.status)
'''


def probe(library: str) -> str:
    env = dict(os.environ, SYN_ROOT=ROOT, SYNAPTIK_NCCL_LIBRARY=library)
    return subprocess.run([sys.executable, "-c", PROBE], env=env, capture_output=True, text=True, check=True, timeout=120).stdout.strip()


def test_a_named_library_that_does_not_load_leaves_the_communicator_unavailable(tmp_path):
    assert probe(str(tmp_path / "libnccl_missing.so")) == "status 15"


def test_the_named_library_is_the_one_bound(tmp_path):
    fake = str(tmp_path / "libfake_nccl.so")
    subprocess.run(["gcc", "-O1", "-shared", "-fPIC", "-o", fake, os.path.join(ROOT, "tests", "fake_nccl.c"), "-ldl"], check=True)
    assert probe(fake) == "id " + bytes(i ^ 0x5a for i in range(128)).hex()

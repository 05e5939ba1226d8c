"""The device-free C++ under AddressSanitizer and UndefinedBehaviorSanitizer.

The reference runs its device-free unit set in an ASan+UBSan build (marfrit/arcint tests/acceptance/cells/sanitizers.sh).
Here the two host-only libraries -- the replay of the kernels' lane code (the very text the GPU runs: decoders, bit
tricks, the GEMV row loop, the all-reduce slot protocol) and the GGUF reader with its malformed-file cases -- are built
with -fsanitize=address,undefined and their suites run again in a child interpreter with the ASan runtime preloaded.
An out-of-bounds read of a block, a shift past the word or a signed overflow in the lane code ends the child non-zero."""
import os
import shutil
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _runtime():
    cc = shutil.which("gcc") or "/usr/bin/gcc"
    if not os.path.exists(cc):
        return None
    p = subprocess.run([cc, "-print-file-name=libasan.so"], capture_output=True, text=True).stdout.strip()
    return p if os.path.isabs(p) and os.path.exists(p) else None


# the mutant builds of the lane code are left out: they are wrong on purpose and a sanitized build of each costs a compile
@pytest.mark.parametrize("suite,select", [("tests/test_emul.py", "not mutants"), ("tests/test_gguf_loader.py", "")])
def test_suite_under_asan_ubsan(suite, select):
    rt = _runtime()
    if rt is None:
        pytest.skip("no ASan runtime beside gcc")
    env = dict(os.environ, B200Q_SANITIZE="1", LD_PRELOAD=rt, ASAN_OPTIONS="detect_leaks=0:abort_on_error=0",
               UBSAN_OPTIONS="halt_on_error=1:print_stacktrace=1")
    r = subprocess.run([sys.executable, "-m", "pytest", suite, "-x", "-q", "-m", "not gpu", "-p", "no:cacheprovider"] + (["-k", select] if select else []), cwd=ROOT, env=env,
                       capture_output=True, text=True, timeout=1500)
    tail = (r.stdout + r.stderr)[-3000:]
    assert r.returncode == 0, tail
    assert "passed" in r.stdout and "AddressSanitizer" not in tail and "runtime error" not in tail, tail

"""Build the C++ host helpers with AddressSanitizer and UndefinedBehaviorSanitizer and run their exerciser.

``python -m ollama_b200.native.sanitize`` compiles ``codecs.cpp``, ``bpe.cpp`` and ``selftest.cc`` into one instrumented program
(``-fsanitize=address,undefined -fno-sanitize-recover=all``), runs it and exits with its status.  The reference relies on the
Go race detector and fuzzing for its host code; the counterpart for C++ that parses model files and tokenises untrusted
text is a sanitizer build that sees every codec and the merge loop on hostile inputs."""
from __future__ import annotations

import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
FLAGS = ["-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", "-ffp-contract=off", "-fsanitize=address,undefined", "-fno-sanitize-recover=all"]


def run(verbose: bool = False) -> int:
    srcs = [os.path.join(HERE, f) for f in ("codecs.cpp", "bpe.cpp", "selftest.cc")]
    with tempfile.TemporaryDirectory() as d:
        exe = os.path.join(d, "selftest_asan")
        r = subprocess.run(["g++", *FLAGS, "-x", "c++", *srcs, "-o", exe, "-lpthread"], capture_output=True, text=True)
        if r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
            return r.returncode
        env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1")
        r = subprocess.run([exe], capture_output=True, text=True, env=env, timeout=600)
        if verbose or r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
        return r.returncode


if __name__ == "__main__":
    sys.exit(run(verbose=True))

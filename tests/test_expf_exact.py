"""emelb::expf_exact (emel.cpp_b200/csrc/expf_exact.h, the source the CUDA kernels compile)
must return the bits of the host C library's expf, the function the reference calls for silu
and for the attention softmax.  Checked on the CPU over a strided sweep of all 2^32 float bit
patterns (stride 1 = every float, about 5 s on 8 cores; the default stride keeps the suite short)."""
import os
import subprocess
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))


def test_expf_exact_matches_host_libm():
    exe = os.path.join(tempfile.gettempdir(), "emelb_expf_harness")
    subprocess.run(["g++", "-O2", "-ffp-contract=off", "-mfma", "-pthread", "-o", exe,
                    os.path.join(HERE, "expf_exact_harness.cc")], check=True)
    stride = os.environ.get("EMELB_EXPF_STRIDE", "5")
    out = subprocess.run([exe, stride], check=True, capture_output=True, text=True)
    assert int(out.stdout.strip()) == 0, out.stderr

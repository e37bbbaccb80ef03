"""The native runtime under ThreadSanitizer and AddressSanitizer: the concurrency check (client threads submitting, streaming,
cancelling and polling against the request engine's actor thread) must verify its own results and draw no sanitizer report."""
import subprocess

import pytest

from tensorrt_edge_llm_b200 import build


@pytest.mark.parametrize("sanitizer", ["thread", "address"])
def test_request_engine_is_clean_under_sanitizer(sanitizer):
    probe = subprocess.run(["g++", f"-fsanitize={sanitizer}", "-x", "c++", "-", "-o", "/dev/null"], input="int main(){return 0;}",
                           text=True, capture_output=True)
    if probe.returncode != 0:
        pytest.skip(f"the toolchain has no {sanitizer} sanitizer runtime")
    exe = build.build_race_check(sanitizer)
    out = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    report = out.stdout + out.stderr
    assert out.returncode == 0, report[-2000:]
    assert "Sanitizer" not in report, report[-4000:]
    assert "mismatches 0" in report and "failed 0" in report

"""Replays the device's weight-tile schedule on the CPU (tests/schedule_sim.cpp includes the same
qmk_schedule.h the kernel is compiled with): every chunk of every weight matrix is fetched exactly once
per phase, in phase order, aligned, for several grid sizes, vocabularies and phase sub-ranges."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_schedule_covers_every_weight_once(tmp_path):
    exe = tmp_path / "schedule_sim"
    subprocess.run(["g++", "-std=c++17", "-O2", "-I", os.path.join(ROOT, "qimeng_megakernel_b200", "csrc"),
                    "-o", str(exe), os.path.join(ROOT, "tests", "schedule_sim.cpp")], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    assert "schedule ok" in out.stdout


def test_batched_schedule_partition_and_slots(tmp_path):
    """The stream-K unit partition of the batched kernel (tests/batch_schedule_sim.cpp includes the same
    qmk_batch_schedule.h): every unit owned once, two scratch slots per CTA suffice, ticket counts match."""
    exe = tmp_path / "batch_schedule_sim"
    subprocess.run(["g++", "-std=c++17", "-O2", "-I", os.path.join(ROOT, "qimeng_megakernel_b200", "csrc"),
                    "-o", str(exe), os.path.join(ROOT, "tests", "batch_schedule_sim.cpp")], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    assert "batch schedule ok" in out.stdout

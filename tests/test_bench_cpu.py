"""Host-side pieces of bench.py that need no GPU: byte accounting, the clock-sample filter and the
reference arm's JSON line (the CPU port on a tiny workload)."""
import datetime
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import bench  # noqa: E402
from mongoose_b200 import configs as mc  # noqa: E402


def test_algorithmic_bytes_of_the_headline_config():
    # 24 layers x 15 841 280 B + lm_head 144 643 072 B of Q8_0 blocks; 12 288 B of fp16 KV per position
    assert mc.weight_bytes_per_token(mc.QWEN25_05B) == 524_833_792
    assert mc.kv_bytes_per_position(mc.QWEN25_05B) == 12_288
    # steps 33..232 of the benchmark window: mean context 132.5
    assert bench.algorithmic_bytes_per_token(mc.QWEN25_05B, 32, 200) == 526_461_952
    assert mc.weight_bytes_per_token(mc.QWEN25_7B) == 7_512_178_688


class FakeSmi:
    def __init__(self, lines):
        self.lines = lines

    def terminate(self):
        pass

    def communicate(self, timeout=None):
        return "\n".join(self.lines), ""


def smi_line(t, mhz, power, reasons=("Not Active",) * 4):
    ts = t.strftime("%Y/%m/%d %H:%M:%S.%f")[:-3]
    return f"{ts}, {mhz}, 1965, {power}, 0x0, " + ", ".join(reasons)


def test_clock_samples_are_kept_only_inside_the_timed_region():
    now = datetime.datetime.now()
    ms = lambda d: now + datetime.timedelta(milliseconds=d)   # noqa: E731
    cs = bench.ClockSampler(0)
    cs.proc = FakeSmi([smi_line(ms(-900), 345, 90.0),                       # idle, long before the region
                       smi_line(ms(-80), 1965, 400.0),
                       smi_line(ms(-60), 1950, 410.0, ("Not Active", "Not Active", "Not Active", "Active")),
                       smi_line(ms(-40), 1965, 405.0),
                       smi_line(ms(+400), 300, 80.0),                       # after the region
                       "garbage line"])
    cs.windows = [[ms(-90), ms(-30)]]
    got = cs.stop()
    assert got["samples"] == 3 and got["sm_mhz"] == 1965.0 and got["sm_max_mhz"] == 1965.0
    assert got["power_w_max"] == 410.0 and got["reasons"] == ["sw_power_cap"]
    assert "window" not in got


def test_clock_brackets_widen_when_nvidia_smi_is_slower_than_the_timed_region():
    now = datetime.datetime.now()
    ms = lambda d: now + datetime.timedelta(milliseconds=d)   # noqa: E731
    cs = bench.ClockSampler(0)
    cs.proc = FakeSmi([smi_line(ms(-900), 345, 90.0), smi_line(ms(-160), 1965, 300.0), smi_line(ms(+60), 1935, 310.0),
                       smi_line(ms(+2500), 300, 80.0)])
    cs.windows = [[ms(-90), ms(-30)], [ms(-20), ms(0)]]       # two timed regions, no sample inside either
    got = cs.stop()
    assert got["samples"] == 2 and got["sm_mhz"] == 1950.0 and "widened by 100 ms" in got["window"]


def test_clock_sampler_without_nvidia_smi_reports_so():
    cs = bench.ClockSampler(0)
    assert cs.stop()["reasons"] == ["nvidia-smi unavailable"]


def test_reference_arm_prints_the_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload",
                          "tiny-q8_0-b1", "--steps", "4", "--warmup", "1"],
                         capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "decode_tokens_per_s" and line["unit"] == "tok/s"
    assert line["value"] > 0 and line["higher_is_better"] is True
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["config"]["workload"] == "tiny-q8_0-b1"

"""nvidia-smi clock and throttle-reason sampler used while timing (read-only queries)."""
import statistics
import subprocess
import threading
import time


class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self.proc, self.marks = index, [], None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        threading.Thread(target=self._read, daemon=True).start()

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def mark(self, t0, t1):
        self.marks.append((t0, t1))

    def stop(self):
        if self.proc is None:
            return None
        time.sleep(0.15)
        self.proc.terminate()
        rows = [(t, [x.strip() for x in s.split(",")]) for t, s in self.samples if s]
        rows = [(t, r) for t, r in rows if len(r) >= 6 and r[0].isdigit()]
        if not rows:
            return None
        inside = [r for t, r in rows if any(a - 0.05 <= t <= b + 0.05 for a, b in self.marks)] or [r for _, r in rows]
        reasons = []
        for name, col in (("hw_slowdown", 2), ("hw_thermal_slowdown", 3), ("sw_thermal_slowdown", 4),
                          ("sw_power_cap", 5)):
            if any(r[col].lower().startswith("active") for r in inside):
                reasons.append(name)
        return {"sm_mhz": statistics.median(int(r[0]) for r in inside), "sm_max_mhz": int(inside[0][1]),
                "reasons": reasons, "samples": len(inside)}

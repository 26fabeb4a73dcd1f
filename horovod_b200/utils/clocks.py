"""GPU clock record for benchmark lines: one ``nvidia-smi`` process samples SM
clock, power and throttle reasons every 100 ms with timestamps for the whole
run; each measurement asks for the summary of its own time window. Reading
only: nothing here changes a GPU setting."""
import datetime
import statistics
import subprocess
import threading
import time

_QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,"
          "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
          "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
_REASONS = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")


class ClockLog:
    def __init__(self, device_index, period_ms=100):
        self.samples = []  # (unix time, sm MHz, max MHz, watts, set of reasons)
        self._lock = threading.Lock()
        self._proc = None
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(device_index), "--query-gpu=" + _QUERY,
                 "--format=csv,noheader,nounits", "-lms", str(period_ms)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self._thread = threading.Thread(target=self._read, daemon=True)
        self._thread.start()

    def _read(self):
        for line in self._proc.stdout:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 8:
                continue
            try:
                t = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                sm, smax, watts = float(f[1]), float(f[2]), float(f[3])
            except ValueError:
                continue
            reasons = {n for n, v in zip(_REASONS, f[4:8]) if v.lower().startswith("active")}
            with self._lock:
                self.samples.append((t, sm, smax, watts, reasons))

    def window(self, t0, t1):
        """Summary of the samples taken between two ``time.time()`` values (the
        nearest sample when the window is shorter than the sampling period)."""
        if self._proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.0)
        with self._lock:
            all_samples = list(self.samples)
        inside = [s for s in all_samples if t0 <= s[0] <= t1]
        if not inside and all_samples:
            mid = 0.5 * (t0 + t1)
            inside = [min(all_samples, key=lambda s: abs(s[0] - mid))]
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no sample"]}
        reasons = set()
        for s in inside:
            reasons |= s[4]
        return {"sm_mhz": statistics.median(s[1] for s in inside), "sm_max_mhz": inside[-1][2],
                "power_w": round(max(s[3] for s in inside), 1), "reasons": sorted(reasons),
                "samples": len(inside)}

    def stop(self):
        if self._proc is not None:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()

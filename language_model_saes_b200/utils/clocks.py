"""Clock, power and throttle-reason sampling of one GPU while a timed region runs (read-only NVML queries from a thread,
``nvidia-smi -lms`` as the fall-back). Used by ``bench.py`` and by the micro-benchmarks so that every reported time
comes with the SM clock it was measured at and with the reasons, if any, for which the clock was held down."""

from __future__ import annotations

import statistics
import subprocess
import threading
import time


class ClockSampler:
    """Samples SM clock, power and clock-event (throttle) reasons of this rank's GPU while the timed region runs.
    NVML is polled from a thread every few milliseconds (read-only queries), so that even a 50 ms region yields
    samples; without the NVML bindings it falls back to ``nvidia-smi -lms``."""

    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, gpu_index: int, period_s: float = 0.02):
        self.gpu = gpu_index
        self.period = period_s
        self.samples: list[tuple[float, float, int]] = []  # (sm MHz, watts, reason bits)
        self.sm_max = None
        self._stop = threading.Event()
        self._thread = None
        self._smi = None

    def _nvml_handle(self):
        import pynvml
        import torch

        pynvml.nvmlInit()
        uuid = getattr(torch.cuda.get_device_properties(self.gpu), "uuid", None)
        if uuid is not None:
            try:
                return pynvml, pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + str(uuid)).encode())
            except Exception:  # noqa: BLE001
                pass
        return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.gpu)

    def start(self):
        try:
            nv, h = self._nvml_handle()
            self.sm_max = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons

            def poll():
                while not self._stop.is_set():
                    try:
                        self.samples.append((float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)),
                                             nv.nvmlDeviceGetPowerUsage(h) / 1000.0, int(reasons(h))))  # fmt: skip
                    except Exception:  # noqa: BLE001
                        pass
                    time.sleep(self.period)

            self._thread = threading.Thread(target=poll, daemon=True)
            self._thread.start()
            # the first queries of a process are slow (the library sets itself up) and the management library and kernel
            # launches share locks in the driver: let them happen here, before the timed region opens
            t0 = time.perf_counter()
            while len(self.samples) < 2 and time.perf_counter() - t0 < 2.0:
                time.sleep(0.005)
        except Exception:  # noqa: BLE001 - no NVML bindings: nvidia-smi
            self._start_smi()

    def _start_smi(self):
        fields = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
        try:
            self._smi = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={fields}", "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)  # fmt: skip

            def read():
                for line in self._smi.stdout:
                    c = [x.strip() for x in line.split(",")]
                    if len(c) >= 7 and c[0].replace(".", "").isdigit():
                        bits = sum(v for (n, v), col in zip(self.REASONS.items(), c[3:7]) if col.lower().startswith("active"))
                        self.samples.append((float(c[0]), float(c[2] or 0), bits))
                        self.sm_max = float(c[1])

            threading.Thread(target=read, daemon=True).start()
        except OSError:
            self._smi = None

    def stop(self) -> dict:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=1.0)
        if self._smi is not None:
            time.sleep(0.1)
            self._smi.terminate()
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": ["no samples"]}
        busy = [s for s in self.samples if s[1] > 300] or self.samples
        bits = 0
        for s in self.samples:
            bits |= s[2]
        return {
            "sm_mhz": statistics.median(s[0] for s in busy),
            "sm_max_mhz": self.sm_max,
            "power_w_max": max(s[1] for s in self.samples),
            "samples": len(self.samples),
            "reasons": [n for n, v in self.REASONS.items() if bits & v],
        }

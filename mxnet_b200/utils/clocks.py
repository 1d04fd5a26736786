"""Background sampler of GPU clocks and throttle reasons (read-only NVML queries) used by the
benchmark to attach a ``clocks`` record to every measurement."""
import threading
import time


class ClockSampler(object):
    def __init__(self, index=0, interval=0.2):
        self.index, self.interval = index, interval
        self.samples = []
        self.reasons = set()
        self.max_sm = None
        self._stop = False
        self._thread = None
        self._nvml = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_sm = pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM)
        except Exception:  # pylint: disable=broad-except
            self._nvml = None
            return self
        self._stop = False
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()
        return self

    def _loop(self):
        n = self._nvml
        names = {'hw_slowdown': getattr(n, 'nvmlClocksThrottleReasonHwSlowdown', 0x8),
                 'hw_thermal_slowdown': getattr(n, 'nvmlClocksThrottleReasonHwThermalSlowdown', 0x40),
                 'sw_thermal_slowdown': getattr(n, 'nvmlClocksThrottleReasonSwThermalSlowdown', 0x20),
                 'sw_power_cap': getattr(n, 'nvmlClocksThrottleReasonSwPowerCap', 0x4)}
        while not self._stop:
            try:
                sm = n.nvmlDeviceGetClockInfo(self._handle, n.NVML_CLOCK_SM)
                util = n.nvmlDeviceGetUtilizationRates(self._handle).gpu
                self.samples.append((sm, util))
                mask = n.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:  # pylint: disable=broad-except
                pass
            time.sleep(self.interval)

    def stop(self):
        self._stop = True
        if self._thread is not None:
            self._thread.join(timeout=2)
        loaded = sorted(s for s, u in self.samples if u >= 50) or sorted(s for s, _ in self.samples)
        med = loaded[len(loaded) // 2] if loaded else None
        return {'sm_mhz': med, 'sm_max_mhz': self.max_sm, 'reasons': sorted(self.reasons), 'samples': len(self.samples)}

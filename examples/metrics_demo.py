"""Metrics without a server: counters, histograms, the request-rate tracker and aggregator, Prometheus text
(reference: examples/metrics_demo.rs)."""
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from oxibonsai_b200.runtime.metrics import InferenceMetrics, RequestRateTracker

m = InferenceMetrics()
for request in range(3):
    m.requests.inc()
    m.prompt_tokens.inc(40 + request)
    tracker = RequestRateTracker()
    t0 = time.perf_counter()
    for token in range(16):
        time.sleep(0.001)                       # stands in for a decode step
        tracker.on_token()
        m.tokens_generated.inc()
        m.decode_token_seconds.observe(0.001)
    m.request_seconds.observe(time.perf_counter() - t0)
    m.aggregator.record(tracker)
snap = m.aggregator.snapshot()
print(f"requests {snap['completed_requests']}, mean {snap['tokens_per_second']:.0f} tok/s, inter-token p50 {snap['itl_p50'] * 1e3:.2f} ms, "
      f"p95 {snap['itl_p95'] * 1e3:.2f} ms")
print(m.render_prometheus()[:600])

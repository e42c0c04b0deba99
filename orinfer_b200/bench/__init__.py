"""HTTP-level benchmark and acceptance clients for a running ``orinfer serve``.

Every number here is taken from the outside of the server, through the same routes a user
calls, so queueing, prefill, HTTP and detokenisation are inside the measured wall time.  The
measurement definitions follow the reference's tools (tools/bench/concurrency.py,
mixed.py, scheduling.py, startup.py, acceptance.py, output_stress.py, mini_weka_compact.py):

* ``committed_output_tps`` = sum of ``usage.completion_tokens`` / wall time of the round;
* gaps between SSE chunks are *arrival gaps*, not inter-token latency (speculation and
  UTF-8 grouping can put several tokens in one chunk);
* TTFT = time to the first non-empty content / reasoning / tool-call delta.
"""

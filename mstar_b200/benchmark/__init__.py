"""Client-side benchmark harness: synthetic workloads per request type, per-request metrics (time to first chunk per
modality, inter-chunk latency, end-to-end latency, audio real-time factor and streaming viability) and aggregate
throughput, in offline (batches), closed-loop (fixed concurrency) and online (Poisson arrivals) firing modes.

    python -m mstar_b200.benchmark.runner --url http://127.0.0.1:8000 --request-type tts --num-requests 64 \\
        --mode closed_loop --max-concurrency 16 --json results.json
"""

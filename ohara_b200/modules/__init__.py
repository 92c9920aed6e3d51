"""Building blocks: norms, feed-forwards, attention, KV cache, mixture-of-experts, scans."""

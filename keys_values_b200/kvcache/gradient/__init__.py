

def get_replay_logs(gpt_model):
    """Replay logs of all layers after an inference pass with logging switched on
    (``keys_values/kvcache/gradient/inference_replay.py:483-493``)."""
    from keys_values_b200.kvcache.basics import KVCacheWithBuffers

    caches = gpt_model.get_kv_caches()
    if any(c is None or not isinstance(c, KVCacheWithBuffers) for c in caches):
        raise IndexError("All blocks of GPT model must have KV caches of type KVCacheWithBuffers assigned")
    if not all(c._do_replay_log for c in caches):
        raise IndexError("All KV caches of GPT model must have replay logging activated")
    return [c.get_replay_log() for c in caches]

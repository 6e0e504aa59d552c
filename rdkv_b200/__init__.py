"""rdkv_b200 — B200-native packed-KV decode path."""

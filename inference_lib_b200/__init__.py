"""B200-native Hogwild! fragmented-KV attention (drop-in for the ``libhogatt`` torch ops)."""

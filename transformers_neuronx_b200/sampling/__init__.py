from .sampler import MAX_SUPPRESSED, ROW_WORDS, Sampler, needs_top_p, pack_rows

"""The cases of tests/golden/make_golden.py that the tests have to know as well (no import of the
reference here): frequency scalings of the rotary encoding, and (top_k, top_p, temperature) of the
sampler."""
ROPE_SCALINGS = {
    "linear": {"rope_type": "linear", "factor": 4.0},
    "llama3": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
               "original_max_position_embeddings": 8192},
    "yarn": {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 4096},
    "yarn_mscale": {"rope_type": "yarn", "factor": 40.0, "original_max_position_embeddings": 4096, "beta_fast": 32.0,
                    "beta_slow": 1.0, "mscale": 1.0, "mscale_all_dim": 0.5},
    "yarn_factor": {"rope_type": "yarn", "factor": 2.0, "original_max_position_embeddings": 2048,
                    "attention_factor": 1.25, "truncate": False},
}
SAMPLER_CASES = [(0, 1.0, 1.0), (5, 1.0, 1.0), (0, 0.7, 1.0), (8, 0.6, 0.7), (3, 0.999, 1.3), (0, 0.05, 1.0)]

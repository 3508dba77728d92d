"""batchspec_b200: a single-GPU (sm_100a) inference engine for the Llama-3 dense
decoder, assembled from parametrised parts over a paged cache."""
__version__ = "0.1.0"

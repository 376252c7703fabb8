"""CUDA-graph wrapper for the one-token decode step (placeholder, filled in below)."""
def get_graphed_model(model, cache):
    raise NotImplementedError

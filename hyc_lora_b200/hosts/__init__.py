"""Minimal host models that expose the swap points of the reference's model files
(models/modeling_llama.py, modeling_mistral.py, modeling_roberta.py) so that the
operator layer can be exercised end to end on synthetic data.  They are harnesses for
the compression path, not re-implementations of the HF models."""

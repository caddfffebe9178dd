"""Self-contained model zoo with Hugging Face parameter names (see ``common.py``)."""

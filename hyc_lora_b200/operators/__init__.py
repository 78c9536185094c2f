"""Drop-in ``EfficientMemory*`` operator modules (same file and class names as the
reference's ``operators`` package)."""

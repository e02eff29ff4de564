"""Drop-in stand-in for the reference's ``kernels`` package (one module, same import path)."""

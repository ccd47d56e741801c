"""Small user-facing utilities: comparing benchmark records of two engines."""

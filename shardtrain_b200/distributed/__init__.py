"""Rank arithmetic, process-group ownership and NVLink peer memory."""

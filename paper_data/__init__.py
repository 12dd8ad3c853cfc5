"""Measurement records of this build (platform ``b200``); same record schema as the reference project's published data."""

"""Comparator methods evaluated against STAC-R at a matched saved-activation surface or optimizer-state budget."""

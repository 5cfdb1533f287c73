"""Named option sets of the Lattice optimizer.

The reference's presets (``bitlattice/optim/presets.py``: 'muon', 'muon_fast', 'balanced', 'light', 'normuon') all use
Newton-Schulz or factored directions, which are outside this build; the names are kept so that asking for one fails
with an explanation instead of a KeyError.
"""
PRESETS: dict[str, dict] = {}
REFERENCE_PRESETS = ("muon", "muon_fast", "balanced", "light", "normuon")

"""Worst error of each replayed case in a clean run: max |got - want| over every compared logit,
divided by the largest |want| of its step.  ``replay.check_worst`` fails a case that exceeds
twice its figure.  A case that is not listed is only held to the blanket tolerance."""
RECORDED = {
}

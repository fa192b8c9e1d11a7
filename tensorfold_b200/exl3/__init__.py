"""Routed experts on EXL3 trellis-coded weights (mirror of the reference's ``tensorfold.cuda.exl3``)."""

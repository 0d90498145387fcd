"""Sentinel values shared by adapters, backbones and losses.

Same numeric contract as the reference's ``nestor/constants.py:1-3`` so that data
prepared for either stack is interchangeable.
"""

CLS_TOKEN_POS = -1
PADDING_TOKEN_POS = -2
PADDING_TOKEN_VALUE = -100

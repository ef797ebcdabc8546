"""Test oracle for the RNS linear path (not part of the product)."""

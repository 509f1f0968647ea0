"""Test oracle for the W8A8 linear path. TEST INFRASTRUCTURE — the product never imports this."""

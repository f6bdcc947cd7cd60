"""TEST INFRASTRUCTURE — CPU checkers of the token-sampling path. Not imported by the product."""

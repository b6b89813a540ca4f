import unittest

_tc = unittest.TestCase()
assert_raises = _tc.assertRaises
assert_equal = _tc.assertEqual
assert_true = _tc.assertTrue

//! `GkrOps` and `MleOps` (`prover/lookups/gkr_prover.rs:172-220`, `prover/lookups/mle.rs:9-14`).
//!
//! Layers stay on the device between rounds. The sum-check round reads back eight words (the two sums); the
//! univariate polynomial is then built by the reference's own `correct_sum_as_poly_in_first_variable`, as the CPU
//! and SIMD backends do (`cpu/lookups/gkr.rs:39-69`).
use stwo::core::fields::m31::BaseField;
use stwo::core::fields::qm31::SecureField;
use stwo::prover::backend::Column;
use stwo::prover::lookups::gkr_prover::{
    correct_sum_as_poly_in_first_variable, EqEvals, GkrMultivariatePolyOracle, GkrOps, Layer,
};
use stwo::prover::lookups::mle::{Mle, MleOps};
use stwo::prover::lookups::sumcheck::MultivariatePolyOracle;
use stwo::prover::lookups::utils::UnivariatePoly;

use crate::column::{B200SecureColumn, DeviceWords};
use crate::ctx::{check, ctx, B200Backend};
use crate::ffi;
use crate::fri::words;

const GRAND_PRODUCT: i32 = 0;
const LOGUP_GENERIC: i32 = 1;
const LOGUP_MULTIPLICITIES: i32 = 2;
const LOGUP_SINGLES: i32 = 3;

fn secure(w: &[u32]) -> SecureField { SecureField::from_u32_unchecked(w[0], w[1], w[2], w[3]) }

/// (kind, numerators or null, denominators, entries) of a layer, as the library's GKR entry points take them.
fn parts(layer: &Layer<B200Backend>) -> (i32, *const u32, *const u32, usize) {
    match layer {
        Layer::GrandProduct(col) => (GRAND_PRODUCT, std::ptr::null(), col.0.ptr as *const u32, col.len()),
        Layer::LogUpGeneric { numerators, denominators } => {
            (LOGUP_GENERIC, numerators.0.ptr as *const u32, denominators.0.ptr as *const u32, denominators.len())
        }
        Layer::LogUpMultiplicities { numerators, denominators } => {
            (LOGUP_MULTIPLICITIES, numerators.0.ptr as *const u32, denominators.0.ptr as *const u32, denominators.len())
        }
        Layer::LogUpSingles { denominators } => (LOGUP_SINGLES, std::ptr::null(), denominators.0.ptr as *const u32, denominators.len()),
    }
}

impl GkrOps for B200Backend {
    fn gen_eq_evals(y: &[SecureField], v: SecureField) -> Mle<Self, SecureField> {
        let out = DeviceWords::uninit(4usize << y.len());
        let yw: Vec<u32> = y.iter().flat_map(|&q| words(q)).collect();
        check(unsafe { ffi::zkb_gkr_eq_evals(ctx(), yw.as_ptr(), y.len() as i32, words(v).as_ptr(), out.ptr) });
        Mle::new(B200SecureColumn(out))
    }

    fn next_layer(layer: &Layer<Self>) -> Layer<Self> {
        let (kind, num, den, n) = parts(layer);
        assert!(n >= 2, "the output layer has no next layer (gkr_prover.rs:262-275 checks this before calling)");
        let den_out = DeviceWords::uninit(4 * (n / 2));
        if kind == GRAND_PRODUCT {
            check(unsafe { ffi::zkb_gkr_next_layer(ctx(), kind, std::ptr::null(), den, n, std::ptr::null_mut(), den_out.ptr) });
            return Layer::GrandProduct(Mle::new(B200SecureColumn(den_out)));
        }
        let num_out = DeviceWords::uninit(4 * (n / 2));
        check(unsafe { ffi::zkb_gkr_next_layer(ctx(), kind, num, den, n, num_out.ptr, den_out.ptr) });
        Layer::LogUpGeneric {
            numerators: Mle::new(B200SecureColumn(num_out)),
            denominators: Mle::new(B200SecureColumn(den_out)),
        }
    }

    fn sum_as_poly_in_first_variable(h: &GkrMultivariatePolyOracle<'_, Self>, claim: SecureField) -> UnivariatePoly<SecureField> {
        let n_variables = h.n_variables();
        assert!(n_variables != 0);
        let (kind, num, den, n) = parts(&h.input_layer);
        let eq_evals: &EqEvals<Self> = h.eq_evals.as_ref();
        let mut out = [0u32; 8];
        check(unsafe {
            ffi::zkb_gkr_sum(ctx(), kind, num, den, n, eq_evals.0.ptr as *const u32, words(h.lambda).as_ptr(), out.as_mut_ptr())
        });
        let eval_at_0 = secure(&out[0..4]) * h.eq_fixed_var_correction;
        let eval_at_2 = secure(&out[4..8]) * h.eq_fixed_var_correction;
        correct_sum_as_poly_in_first_variable(eval_at_0, eval_at_2, claim, eq_evals.y(), n_variables)
    }
}

impl MleOps<BaseField> for B200Backend {
    fn fix_first_variable(mle: Mle<Self, BaseField>, assignment: SecureField) -> Mle<Self, SecureField> {
        let n = mle.len();
        assert!(n >= 2);
        let out = DeviceWords::uninit(4 * (n / 2));
        check(unsafe { ffi::zkb_mle_fix_m31(ctx(), mle.0.ptr as *const u32, n, words(assignment).as_ptr(), out.ptr) });
        Mle::new(B200SecureColumn(out))
    }
}

impl MleOps<SecureField> for B200Backend {
    fn fix_first_variable(mle: Mle<Self, SecureField>, assignment: SecureField) -> Mle<Self, SecureField> {
        let n = mle.len();
        assert!(n >= 2);
        let out = DeviceWords::uninit(4 * (n / 2));
        check(unsafe { ffi::zkb_mle_fix_qm31(ctx(), mle.0.ptr as *const u32, n, words(assignment).as_ptr(), out.ptr) });
        Mle::new(B200SecureColumn(out))
    }
}

/// One sum-check round for a prover that owns its loop: `Layer::fix_first_variable` (`gkr_prover.rs:354-381`) and the
/// next round's two sums in one launch (`zkb_gkr_fix_and_sum`), instead of the trait's separate calls. Returns the fixed
/// layer and `(sum at 0, sum at 2)` before the eq correction.
pub fn fix_and_sum(
    layer: &Layer<B200Backend>,
    r: SecureField,
    eq_evals: &EqEvals<B200Backend>,
    lambda: SecureField,
) -> (Layer<B200Backend>, SecureField, SecureField) {
    let (kind, num, den, n) = parts(layer);
    assert!(n >= 8);
    let den_out = DeviceWords::uninit(4 * (n / 2));
    let num_out = if kind == LOGUP_GENERIC || kind == LOGUP_MULTIPLICITIES { DeviceWords::uninit(4 * (n / 2)) } else { DeviceWords::uninit(0) };
    let mut out = [0u32; 8];
    check(unsafe {
        ffi::zkb_gkr_fix_and_sum(
            ctx(), kind, num, den, n, words(r).as_ptr(), eq_evals.0.ptr as *const u32, words(lambda).as_ptr(),
            num_out.ptr, den_out.ptr, out.as_mut_ptr(),
        )
    });
    let den_mle = Mle::new(B200SecureColumn(den_out));
    let fixed = match kind {
        GRAND_PRODUCT => Layer::GrandProduct(den_mle),
        LOGUP_SINGLES => Layer::LogUpSingles { denominators: den_mle },
        _ => Layer::LogUpGeneric { numerators: Mle::new(B200SecureColumn(num_out)), denominators: den_mle },
    };
    (fixed, secure(&out[0..4]), secure(&out[4..8]))
}

//! Device columns (`ColumnOps`, `Column`; `prover/backend/mod.rs:39-92`). A column owns its device buffer and frees it
//! on drop; `Clone` is a device-to-device copy (`stwo_cuda/base_field_vec.rs:7-60`). `at` / `set` are 4-byte copies:
//! correctness paths only.
use std::ffi::c_void;

use stwo::core::fields::m31::BaseField;
use stwo::core::fields::qm31::SecureField;
use stwo::core::vcs::blake2_hash::Blake2sHash;
use stwo::prover::backend::{Column, ColumnOps};

use crate::ctx::{check, ctx, B200Backend};
use crate::ffi;

/// `words` 32-bit words on the device.
#[derive(Debug)]
pub struct DeviceWords {
    pub ptr: *mut u32,
    pub words: usize,
}
unsafe impl Send for DeviceWords {}
unsafe impl Sync for DeviceWords {}

impl DeviceWords {
    pub fn uninit(words: usize) -> Self {
        let mut p: *mut c_void = std::ptr::null_mut();
        if words > 0 {
            check(unsafe { ffi::zkb_malloc(ctx(), words * 4, &mut p) });
        }
        Self { ptr: p as *mut u32, words }
    }
    pub fn zeros(words: usize) -> Self {
        let w = Self::uninit(words);
        if words > 0 {
            check(unsafe { ffi::zkb_memset_zero(ctx(), w.ptr as *mut c_void, words * 4) });
        }
        w
    }
    pub fn from_host(src: &[u32]) -> Self {
        let w = Self::uninit(src.len());
        if !src.is_empty() {
            check(unsafe { ffi::zkb_h2d(ctx(), w.ptr as *mut c_void, src.as_ptr() as *const c_void, src.len() * 4) });
        }
        w
    }
    pub fn to_host(&self) -> Vec<u32> {
        let mut v = vec![0u32; self.words];
        if self.words > 0 {
            check(unsafe { ffi::zkb_d2h(ctx(), v.as_mut_ptr() as *mut c_void, self.ptr as *const c_void, self.words * 4) });
        }
        v
    }
    pub fn read(&self, word: usize, n: usize) -> Vec<u32> {
        let mut v = vec![0u32; n];
        check(unsafe { ffi::zkb_d2h(ctx(), v.as_mut_ptr() as *mut c_void, self.ptr.add(word) as *const c_void, n * 4) });
        v
    }
    pub fn write(&mut self, word: usize, src: &[u32]) {
        check(unsafe { ffi::zkb_h2d(ctx(), self.ptr.add(word) as *mut c_void, src.as_ptr() as *const c_void, src.len() * 4) });
    }
    /// The two halves as fresh columns (`split_at_mid`).
    pub fn split(self, unit: usize) -> (Self, Self) {
        let mid = (self.words / unit / 2) * unit;
        let (a, b) = (Self::uninit(mid), Self::uninit(self.words - mid));
        unsafe {
            check(ffi::zkb_d2d(ctx(), a.ptr as *mut c_void, self.ptr as *const c_void, mid * 4));
            check(ffi::zkb_d2d(ctx(), b.ptr as *mut c_void, self.ptr.add(mid) as *const c_void, (self.words - mid) * 4));
        }
        (a, b)
    }
}
impl Clone for DeviceWords {
    fn clone(&self) -> Self {
        let w = Self::uninit(self.words);
        if self.words > 0 {
            check(unsafe { ffi::zkb_d2d(ctx(), w.ptr as *mut c_void, self.ptr as *const c_void, self.words * 4) });
        }
        w
    }
}
impl Drop for DeviceWords {
    fn drop(&mut self) {
        if !self.ptr.is_null() {
            unsafe { ffi::zkb_free(ctx(), self.ptr as *mut c_void) };
        }
    }
}

/// `Col<B200Backend, BaseField>`: one canonical word per element.
#[derive(Clone, Debug)]
pub struct B200BaseColumn(pub DeviceWords);
/// `Col<B200Backend, SecureField>`: four consecutive words per element (the reference's `SecureFieldVec`).
#[derive(Clone, Debug)]
pub struct B200SecureColumn(pub DeviceWords);
/// `Col<B200Backend, Blake2sHash>`: eight words per node.
#[derive(Clone, Debug)]
pub struct B200HashColumn(pub DeviceWords);

impl ColumnOps<BaseField> for B200Backend {
    type Column = B200BaseColumn;
    fn bit_reverse_column(column: &mut Self::Column) {
        let n = column.0.words;
        assert!(n.is_power_of_two());
        check(unsafe { ffi::zkb_bit_reverse_m31(ctx(), column.0.ptr, n.ilog2() as i32) });
    }
}
impl ColumnOps<SecureField> for B200Backend {
    type Column = B200SecureColumn;
    fn bit_reverse_column(column: &mut Self::Column) {
        let n = column.0.words / 4;
        assert!(n.is_power_of_two());
        check(unsafe { ffi::zkb_bit_reverse_qm31(ctx(), column.0.ptr, n.ilog2() as i32) });
    }
}
impl ColumnOps<Blake2sHash> for B200Backend {
    type Column = B200HashColumn;
    fn bit_reverse_column(_column: &mut Self::Column) {
        unimplemented!("hash columns are never bit-reversed by the prover (the CPU and SIMD backends do not implement it either)")
    }
}

impl Column<BaseField> for B200BaseColumn {
    fn zeros(len: usize) -> Self { Self(DeviceWords::zeros(len)) }
    unsafe fn uninitialized(len: usize) -> Self { Self(DeviceWords::uninit(len)) }
    fn to_cpu(&self) -> Vec<BaseField> { self.0.to_host().into_iter().map(BaseField::from_u32_unchecked).collect() }
    fn len(&self) -> usize { self.0.words }
    fn at(&self, index: usize) -> BaseField { BaseField::from_u32_unchecked(self.0.read(index, 1)[0]) }
    fn set(&mut self, index: usize, value: BaseField) { self.0.write(index, &[value.0]) }
    fn batch_at(&self, indices: &[usize]) -> Vec<BaseField> { Self::batch_at_multi(&[self], indices) }
    fn batch_at_multi(columns: &[&Self], indices: &[usize]) -> Vec<BaseField> {
        if columns.is_empty() || indices.is_empty() {
            return Vec::new();
        }
        let ptrs: Vec<*const u32> = columns.iter().map(|c| c.0.ptr as *const u32).collect();
        let idx: Vec<u32> = indices.iter().map(|&i| i as u32).collect();
        let mut out = vec![0u32; ptrs.len() * idx.len()];  // row-major [index][column], as the trait documents
        check(unsafe { ffi::zkb_gather_multi(ctx(), ptrs.as_ptr(), ptrs.len() as i32, idx.as_ptr(), idx.len() as i32, out.as_mut_ptr()) });
        out.into_iter().map(BaseField::from_u32_unchecked).collect()
    }
    fn split_at_mid(self) -> (Self, Self) { let (a, b) = self.0.split(1); (Self(a), Self(b)) }
}
impl FromIterator<BaseField> for B200BaseColumn {
    fn from_iter<T: IntoIterator<Item = BaseField>>(iter: T) -> Self {
        let v: Vec<u32> = iter.into_iter().map(|x| x.0).collect();
        Self(DeviceWords::from_host(&v))
    }
}

impl Column<SecureField> for B200SecureColumn {
    fn zeros(len: usize) -> Self { Self(DeviceWords::zeros(4 * len)) }
    unsafe fn uninitialized(len: usize) -> Self { Self(DeviceWords::uninit(4 * len)) }
    fn to_cpu(&self) -> Vec<SecureField> {
        self.0.to_host().chunks_exact(4).map(|w| SecureField::from_u32_unchecked(w[0], w[1], w[2], w[3])).collect()
    }
    fn len(&self) -> usize { self.0.words / 4 }
    fn at(&self, index: usize) -> SecureField {
        let w = self.0.read(4 * index, 4);
        SecureField::from_u32_unchecked(w[0], w[1], w[2], w[3])
    }
    fn set(&mut self, index: usize, value: SecureField) {
        let a = value.to_m31_array();
        self.0.write(4 * index, &[a[0].0, a[1].0, a[2].0, a[3].0]);
    }
    fn split_at_mid(self) -> (Self, Self) { let (a, b) = self.0.split(4); (Self(a), Self(b)) }
}
impl FromIterator<SecureField> for B200SecureColumn {
    fn from_iter<T: IntoIterator<Item = SecureField>>(iter: T) -> Self {
        let v: Vec<u32> = iter.into_iter().flat_map(|x| x.to_m31_array().map(|m| m.0)).collect();
        Self(DeviceWords::from_host(&v))
    }
}

impl Column<Blake2sHash> for B200HashColumn {
    fn zeros(len: usize) -> Self { Self(DeviceWords::zeros(8 * len)) }
    unsafe fn uninitialized(len: usize) -> Self { Self(DeviceWords::uninit(8 * len)) }
    fn to_cpu(&self) -> Vec<Blake2sHash> {
        self.0.to_host().chunks_exact(8).map(|w| { let mut h = [0u8; 32]; h.copy_from_slice(bytemuck::cast_slice(w)); Blake2sHash(h) }).collect()
    }
    fn len(&self) -> usize { self.0.words / 8 }
    fn at(&self, index: usize) -> Blake2sHash {
        let w = self.0.read(8 * index, 8);
        let mut h = [0u8; 32];
        h.copy_from_slice(bytemuck::cast_slice(&w));
        Blake2sHash(h)
    }
    fn set(&mut self, index: usize, value: Blake2sHash) { self.0.write(8 * index, bytemuck::cast_slice(&value.0)) }
    fn split_at_mid(self) -> (Self, Self) { let (a, b) = self.0.split(8); (Self(a), Self(b)) }
}
impl FromIterator<Blake2sHash> for B200HashColumn {
    fn from_iter<T: IntoIterator<Item = Blake2sHash>>(iter: T) -> Self {
        let v: Vec<u32> = iter.into_iter().flat_map(|h| bytemuck::cast::<[u8; 32], [u32; 8]>(h.0)).collect();
        Self(DeviceWords::from_host(&v))
    }
}
